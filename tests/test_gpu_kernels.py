"""Each kernel alone against a plain torch fp32 restatement of the same operation, at sizes
other than the engine's tiny models (odd widths, tails, several pages, grouped heads)."""
import ctypes
import math

import pytest
import torch

from nimbus_infer_rs_b200.cache import PAGE, LayerKV
from nimbus_infer_rs_b200.csrc import ops as ops_mod
from nimbus_infer_rs_b200.engine.batch import build_layout

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    return ops_mod.backend()


def test_library_is_loaded_from_the_tree(ops):
    from nimbus_infer_rs_b200.csrc import build
    assert ops.lib.nb_abi_version() >= 1
    assert build.build().name == "libnimbus_b200.so"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d", [48, 100, 768, 1600])
def test_embed_pos(ops, dtype, d):
    torch.manual_seed(0)
    V, Pn, n = 301, 77, 19
    wte = torch.randn(V, d, device=DEV).to(dtype)
    wpe = torch.randn(Pn, d, device=DEV).to(dtype)
    tok = torch.randint(0, V, (n,), device=DEV, dtype=torch.int32)
    pos = torch.randint(0, Pn, (n,), device=DEV, dtype=torch.int32)
    tok[5] = -1                                   # a padding row
    out = torch.full((n, d), 9.0, device=DEV)
    ops.embed_pos(tok, pos, wte, wpe, out)
    ref = wte[tok.clamp(min=0).long()].float() + wpe[pos.long()].float()
    ref[5] = 0
    assert torch.equal(out, ref)
    ops.embed_pos(tok, pos, wte, None, out)
    ref = wte[tok.clamp(min=0).long()].float()
    ref[5] = 0
    assert torch.equal(out, ref)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d, eps", [(17, 1e-5), (100, 1e-6), (768, 1e-5), (1600, 3e-5), (5000, 1e-5)])
def test_layernorm(ops, out_dtype, d, eps):
    torch.manual_seed(1)
    n = 23
    x = torch.randn(n, d, device=DEV) * 3 + 0.7
    x[3] *= 1e3                                    # large mean and spread
    g = torch.randn(d, device=DEV)
    b = torch.randn(d, device=DEV)
    out = torch.empty(n, d, device=DEV, dtype=out_dtype)
    ops.layernorm(x, g, b, eps, out)
    xd = x.double()
    mean = xd.mean(-1, keepdim=True)
    var = ((xd - mean) ** 2).mean(-1, keepdim=True)
    ref = (xd - mean) / torch.sqrt(var + eps) * g.double() + b.double()
    tol = 1e-5 if out_dtype == torch.float32 else 8e-3
    assert ((out.double() - ref).abs() <= tol * (1 + ref.abs())).all()
    # row selection, with a padding entry
    rows = torch.tensor([4, -1, 0, 22], device=DEV, dtype=torch.int32)
    sel = torch.empty(4, d, device=DEV, dtype=out_dtype)
    ops.layernorm(x, g, b, eps, sel, rows)
    assert torch.equal(sel[0], out[4]) and torch.equal(sel[2], out[0]) and torch.equal(sel[3], out[22])
    assert (sel[1] == 0).all()


def _gelu(y, act):
    if act == 1:
        return 0.5 * y * (1 + torch.tanh(0.7978845608028654 * (y + 0.044715 * y ** 3)))
    if act == 2:
        return 0.5 * y * (1 + torch.erf(y / math.sqrt(2.0)))
    return y


LINEAR_SHAPES = [(1, 64, 64), (5, 1001, 96), (33, 130, 100), (130, 257, 72), (64, 768, 3072),
                 (300, 2304, 768), (7, 50257, 64), (2048, 96, 320), (260, 333, 70), (513, 1000, 100)]


@pytest.mark.parametrize("M, N, K", LINEAR_SHAPES)
@pytest.mark.parametrize("xdt, wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                      (torch.bfloat16, torch.float32)])
def test_linear_against_float64(ops, M, N, K, xdt, wdt):
    torch.manual_seed(M * 7 + N)
    x = torch.randn(M, K, device=DEV).to(xdt)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(wdt)
    bias = torch.randn(N, device=DEV)
    ref0 = x.double() @ w.double().t()
    scale = float(ref0.abs().max())
    tol = 3e-6 * scale * math.sqrt(K / 64)          # fp32 accumulation of K exact products
    # plain product, fp32 out
    out = torch.empty(M, N, device=DEV)
    ops.linear(x, w, None, out)
    assert (out.double() - ref0).abs().max() <= tol
    # bias + activation, output in the activation type
    for act in (1, 2):
        ref = _gelu(ref0 + bias.double(), act)
        o = torch.empty(M, N, device=DEV, dtype=xdt)
        ops.linear(x, w, bias, o, act)
        t = tol if xdt == torch.float32 else tol + 8e-3 * float(ref.abs().max())
        assert (o.double() - ref).abs().max() <= t
    # bias + residual, in place on the fp32 stream
    res = torch.randn(M, N, device=DEV)
    ref = ref0 + bias.double() + res.double()
    stream = res.clone()
    ops.linear(x, w, bias, stream, 0, stream)
    assert (stream.double() - ref).abs().max() <= tol + 1e-6 * float(ref.abs().max())


@pytest.mark.parametrize("M, N, K, out_dtype", [
    (45, 4800, 1600, torch.bfloat16), (192, 4800, 1600, torch.bfloat16), (192, 1600, 6400, torch.float32),
    (64, 768, 768, torch.float32), (130, 20001, 1600, torch.float32), (700, 2304, 776, torch.bfloat16),
    (128, 6400, 1600, torch.bfloat16)])
def test_tensor_core_products_again_and_again(ops, M, N, K, out_dtype):
    """The tiled tensor-core product with its two MMA-issuing threads (a CTA with one tile and
    a long K) and its producer lanes that share the ring's stages: K of 25 and 100 blocks (no
    multiple of the lanes or the stages), rings of 3, 4, 6 and 8 stages, one tile per CTA and
    CTAs that walk over many tiles.  Forty launches back to back, each overlapping the end of
    the one before: every result must be the first one bit for bit (a stage handed out too
    early shows as a difference that depends on timing), and the first one right."""
    torch.manual_seed(N + K)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    bias = torch.randn(N, device=DEV)
    ref = x.double() @ w.double().t() + bias.double()
    was = ops.use_rows
    ops.use_rows = 0                         # the tiled kernel, also where the few-rows kernel would be taken
    try:
        outs = [torch.full((M, N), 3.0, device=DEV, dtype=out_dtype) for _ in range(40)]
        for o in outs:
            ops.linear(x, w, bias, o)
        ops.check_device_errors()
    finally:
        ops.use_rows = was
    tol = 3e-6 * float(ref.abs().max()) * math.sqrt(K / 64)
    if out_dtype == torch.bfloat16:
        tol += 8e-3 * float(ref.abs().max())
    assert (outs[0].double() - ref).abs().max() <= tol
    for i, o in enumerate(outs[1:], 1):
        assert torch.equal(o, outs[0]), f"launch {i} differs from the first"


ROWS_SHAPES = [(64, 2304, 768), (64, 768, 3072), (17, 130, 72), (33, 1000, 100 * 8), (48, 768, 768),
               (100, 1600, 1600), (128, 4800, 1600), (80, 257 * 8, 6400), (20, 333, 64), (128, 128, 8)]


@pytest.mark.parametrize("M, N, K", ROWS_SHAPES)
@pytest.mark.parametrize("split", [0, 1, 2, 3, 5, 8])
def test_products_of_17_to_128_rows(ops, M, N, K, split):
    """The tensor-core kernel whose 128-row operand is the weights: K cut among the CTAs of a
    cluster (the size it chooses, and sizes forced here: one CTA, a size that does not divide
    the rows or the K blocks evenly, the largest), the sums dealt back through distributed
    shared memory.  Rows that are no multiple of 16, columns that are no multiple of 128, a K
    of one block and of a hundred; bias, GELU, the residual added in place, bf16 and fp32
    results; all against float64, and twice, so that what one launch leaves in shared or tensor
    memory cannot help the next."""
    assert ops.use_rows and ops.lib.nb_gemm_tc_rows_supported(M, N, K)
    assert ops.lib.nb_gemm_tc_rows_preferred(64, 768, 3072) and not ops.lib.nb_gemm_tc_rows_preferred(64, 2304, 768)
    plan = (ctypes.c_int * 6)()
    was, was_rows = ops.lib.nb_gemm_tc_rows_force_split(split), ops.use_rows
    ops.use_rows = 2                      # wherever it applies, not only where it is the faster one
    try:
        if not ops.lib.nb_gemm_tc_rows_plan(M, N, K, plan):
            pytest.skip("this cluster size leaves a CTA without a block of K, or the launch does not fit")
        assert split == 0 or plan[1] == split
        torch.manual_seed(M + N + K)
        x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
        w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
        bias = torch.randn(N, device=DEV)
        ref0 = x.double() @ w.double().t()
        tol = 3e-6 * float(ref0.abs().max()) * math.sqrt(max(K, 64) / 64)
        for attempt in range(2):
            before = ops.launches
            out = torch.full((M, N), 9.0, device=DEV)
            ops.linear(x, w, None, out)
            assert ops.launches == before + 1
            assert (out.double() - ref0).abs().max() <= tol
            ref = _gelu(ref0 + bias.double(), 1)
            o = torch.full((M, N), 9.0, device=DEV, dtype=torch.bfloat16)
            ops.linear(x, w, bias, o, 1)
            assert (o.double() - ref).abs().max() <= tol + 8e-3 * float(ref.abs().max())
            res = torch.randn(M, N, device=DEV)
            stream = res.clone()
            ops.linear(x, w, bias, stream, 0, stream)
            ref = ref0 + bias.double() + res.double()
            assert (stream.double() - ref).abs().max() <= tol + 1e-6 * float(ref.abs().max())
        ops.check_device_errors()
    finally:
        ops.lib.nb_gemm_tc_rows_force_split(was)
        ops.use_rows = was_rows


def _paged_cache(n_seqs, lens, Hk, hd, dtype, seed, extra_pages=3, page=PAGE, stale_nan=False):
    """A cache with shuffled pages, filled with random keys/values for the given lengths; what
    lies in the unused part of every page is random too, or (``stale_nan``) not a number."""
    g = torch.Generator().manual_seed(seed)
    max_pages = max(-(-l // page) for l in lens) + 1
    n_pages = sum(-(-l // page) for l in lens) + extra_pages
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.zeros(n_seqs + 2, max_pages, dtype=torch.int32)
    k = torch.randn(n_pages, Hk, page, hd, generator=g).to(dtype)     # stale data everywhere
    v = torch.randn(n_pages, Hk, page, hd, generator=g).to(dtype)
    if stale_nan:
        k.fill_(float("nan"))
        v.fill_(float("nan"))
        v[::2] = float("inf")
    dense_k, dense_v = [], []
    it = iter(perm)
    for s, l in enumerate(lens):
        ks = torch.randn(l, Hk, hd, generator=g).to(dtype)
        vs = torch.randn(l, Hk, hd, generator=g).to(dtype)
        dense_k.append(ks)
        dense_v.append(vs)
        for p in range(-(-l // page)):
            pg = next(it)
            table[s + 1, p] = pg                                        # slot = s + 1
            n = min(page, l - p * page)
            k[pg, :, :n] = ks[p * page:p * page + n].transpose(0, 1)
            v[pg, :, :n] = vs[p * page:p * page + n].transpose(0, 1)
    kv = LayerKV(k.to(DEV), v.to(DEV), table.to(DEV), page, Hk, hd)
    return kv, dense_k, dense_v


def _attention_ref(q, ks, vs, pos, scale, group, window=0):
    """q [H, hd] at position pos over dense keys/values [len, Hk, hd] (float64)."""
    lo = max(0, pos + 1 - window) if window > 0 else 0
    out = []
    for h in range(q.shape[0]):
        kk = ks[lo:pos + 1, h // group].double()
        vv = vs[lo:pos + 1, h // group].double()
        s = (kk @ q[h].double()) * scale
        p = torch.softmax(s, 0)
        out.append(p @ vv)
    return torch.stack(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, Hk, hd, window", [(4, 4, 16, 0), (6, 2, 48, 0), (12, 12, 64, 0),
                                               (5, 1, 128, 0), (3, 3, 32, 70), (2, 2, 256, 0),
                                               (25, 25, 64, 0)])
def test_attention_over_paged_cache(ops, dtype, H, Hk, hd, window):
    """Prefill-like chunks and single decode rows in one launch, sequences of unequal length
    spanning several shuffled pages, with stale data in the unused part of every page."""
    lens = [200, 1, 64, 65, 333]
    new = [200, 1, 3, 1, 40]                     # rows of this step: the last `new` positions
    kv, dk, dv = _paged_cache(len(lens), lens, Hk, hd, dtype, seed=H * 100 + hd)
    entries = [(s + 1, [0] * n, []) for s, n in enumerate(new)]
    pos0 = [l - n for l, n in zip(lens, new)]
    lay = build_layout(entries, pos0, DEV, pad_rows_to=8)
    torch.manual_seed(5)
    width = (H + 2 * Hk) * hd
    qkv = torch.randn(lay.n_rows, width, device=DEV).to(dtype)
    out = torch.full((lay.n_rows, H * hd), 7.0, device=DEV, dtype=dtype)
    scale = 0.37 / math.sqrt(hd)
    ops.attention(qkv, 0, lay, kv, H, out, scale, window)
    r = 0
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    for s, n in enumerate(new):
        for i in range(n):
            q = qkv[r, :H * hd].view(H, hd).cpu()
            ref = _attention_ref(q, dk[s], dv[s], pos0[s] + i, scale, H // Hk, window)
            got = out[r].view(H, hd).double().cpu()
            assert (got - ref).abs().max() <= tol * max(1.0, float(ref.abs().max())), (s, i)
            r += 1
    assert (out[r:] == 0).all()                  # padding rows give zeros


def _check_attention(ops, kv, dk, dv, lens, new, H, Hk, hd, dtype, window=0, seed=5):
    entries = [(s + 1, [0] * n, []) for s, n in enumerate(new)]
    pos0 = [l - n for l, n in zip(lens, new)]
    lay = build_layout(entries, pos0, DEV, pad_rows_to=8)
    torch.manual_seed(seed)
    qkv = torch.randn(lay.n_rows, (H + 2 * Hk) * hd, device=DEV).to(dtype)
    out = torch.full((lay.n_rows, H * hd), 7.0, device=DEV, dtype=dtype)
    scale = 0.37 / math.sqrt(hd)
    ops.attention(qkv, 0, lay, kv, H, out, scale, window)
    assert torch.isfinite(out.float()).all()
    r = 0
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    for s, n in enumerate(new):
        for i in range(n):
            q = qkv[r, :H * hd].view(H, hd).cpu()
            ref = _attention_ref(q, dk[s], dv[s], pos0[s] + i, scale, H // Hk, window)
            got = out[r].view(H, hd).double().cpu()
            assert (got - ref).abs().max() <= tol * max(1.0, float(ref.abs().max())), (s, i)
            r += 1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, Hk, hd", [(4, 4, 32), (6, 2, 48), (12, 12, 64), (2, 1, 128)])
def test_what_an_earlier_owner_left_in_a_page_never_reaches_a_result(ops, dtype, H, Hk, hd):
    """Every row of every page that holds no key of its sequence is NaN (keys) and NaN or
    infinity (values), as if an earlier owner of the page had overflowed.  A masked score is
    replaced, but a probability of zero times such a value is NaN unless the kernel keeps the
    value out: the results must be finite and equal to the reference's, in single decode rows
    (the split decode kernel), in chunks (the mma.sync and the tensor-core prefill kernels,
    by head size) and in 32-bit."""
    lens = [200, 1, 64, 65, 333, 130]
    kv, dk, dv = _paged_cache(len(lens), lens, Hk, hd, dtype, seed=H + hd, stale_nan=True)
    _check_attention(ops, kv, dk, dv, lens, [1] * len(lens), H, Hk, hd, dtype)          # decode
    _check_attention(ops, kv, dk, dv, lens, [200, 1, 3, 65, 40, 130], H, Hk, hd, dtype)   # chunks
    ops.check_device_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_cache_with_another_page_size_takes_the_generic_kernel(ops, dtype):
    """The fast attention kernels are written for pages of 64 tokens and say so
    (`nb_attention_*_supported` return 0 for another page size); the dispatcher then takes the
    generic kernel, which reads any page size: same results, decode rows and chunks."""
    H, Hk, hd, page = 4, 2, 64, 32
    code = 0 if dtype == torch.float32 else 1
    assert not ops.lib.nb_attention_decode_supported(code, hd, H, Hk, page)
    assert ops.lib.nb_attention_decode_supported(code, hd, H, Hk, PAGE)
    assert not ops.lib.nb_attention_prefill_supported(1, hd, H, Hk, page, (H + 2 * Hk) * hd, 0)
    assert not ops.lib.nb_attention_prefill_tc_supported(1, hd, H, Hk, page, (H + 2 * Hk) * hd, 0, 1, H * hd)
    lens = [100, 1, 32, 33, 70]
    kv, dk, dv = _paged_cache(len(lens), lens, Hk, hd, dtype, seed=9, page=page)
    before = ops.launches
    _check_attention(ops, kv, dk, dv, lens, [1] * len(lens), H, Hk, hd, dtype)
    _check_attention(ops, kv, dk, dv, lens, [100, 1, 2, 33, 8], H, Hk, hd, dtype)
    assert ops.launches - before == 2          # one generic launch each, no append pass


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("lens, new", [([450, 129, 128, 64, 1, 391], [450, 128, 1, 64, 1, 300]),
                                       ([1100, 70, 600], [1100, 6, 131])])
@pytest.mark.parametrize("H, Hk, hd, window", [(12, 12, 64, 0), (8, 2, 64, 70), (4, 1, 128, 0),
                                               (2, 2, 128, 150), (3, 3, 64, 1)])
def test_tensor_core_prefill_attention(ops, H, Hk, hd, window, lens, new, out_dtype):
    """The tcgen05 prefill kernel (bf16, head size 64 or 128): chunks of many rows that start
    anywhere in a page, several 128-row tiles per sequence with a ragged last one, grouped
    heads, windows that end inside a page, stale data in every page, the pages of a tile cut
    into one to four runs that are merged (`new` are the rows of this step: the last
    positions of each sequence); and no wait timed out."""
    kv, dk, dv = _paged_cache(len(lens), lens, Hk, hd, torch.bfloat16, seed=H * 10 + hd + window)
    entries = [(s + 1, [0] * n, []) for s, n in enumerate(new)]
    pos0 = [l - n for l, n in zip(lens, new)]
    lay = build_layout(entries, pos0, DEV, pad_rows_to=8)
    assert not lay.is_decode
    torch.manual_seed(6)
    qkv = torch.randn(lay.n_rows, (H + 2 * Hk) * hd, device=DEV).to(torch.bfloat16)
    out = torch.full((lay.n_rows, H * hd), 7.0, device=DEV, dtype=out_dtype)
    scale = 0.6 / math.sqrt(hd)
    ops.attention(qkv, 0, lay, kv, H, out, scale, window)
    ops.check_device_errors()
    r = 0
    for s, n in enumerate(new):
        q = qkv[r:r + n, :H * hd].view(n, H, hd).double().cpu()
        k, v = dk[s].double(), dv[s].double()                     # [len, Hk, hd]
        qpos = torch.arange(pos0[s], pos0[s] + n)[:, None]
        key = torch.arange(lens[s])[None, :]
        vis = key <= qpos
        if window > 0:
            vis &= key > qpos - window
        for h in range(H):
            sc = (q[:, h] @ k[:, h // (H // Hk)].t()) * scale
            sc = sc.masked_fill(~vis, float("-inf"))
            ref = torch.softmax(sc, dim=1) @ v[:, h // (H // Hk)]
            got = out[r:r + n, h * hd:(h + 1) * hd].double().cpu()
            err = (got - ref).abs().max(dim=1).values
            assert err.max() <= 1.5e-2 * max(1.0, float(ref.abs().max())), \
                f"sequence {s}, head {h}, worst row {int(err.argmax())}"
        r += n
    assert (out[r:] == 0).all()                  # padding rows give zeros


@pytest.mark.parametrize("H, Hk, hd, window", [(12, 12, 64, 0), (8, 2, 64, 100), (4, 2, 128, 0)])
def test_tensor_core_prefill_attention_appends_its_own_keys_and_values(ops, H, Hk, hd, window):
    """Sequences whose cached length is a whole number of pages (0, 64, 192): the kernel must
    read the step's keys and values from the step's rows, not from the cache (which holds
    other data there), give what append-then-attend gives, and leave the same cache behind."""
    lens = [450, 128, 64 + 70, 192 + 300, 1]
    pos0 = [0, 0, 64, 192, 0]
    new = [l - p for l, p in zip(lens, pos0)]
    kv_true, dk, dv = _paged_cache(len(lens), lens, Hk, hd, torch.bfloat16, seed=H + hd + window)
    k_stale, v_stale = kv_true.k.clone(), kv_true.v.clone()
    table = kv_true.block_table.cpu()
    for s, (l, p) in enumerate(zip(lens, pos0)):          # spoil the cache where new tokens go
        for pos in range(p, l):
            page = int(table[s + 1, pos // PAGE])
            k_stale[page, :, pos % PAGE] = 9.0
            v_stale[page, :, pos % PAGE] = -9.0
    kv = LayerKV(k_stale, v_stale, kv_true.block_table, PAGE, Hk, hd)
    entries = [(s + 1, [0] * n, []) for s, n in enumerate(new)]
    lay = build_layout(entries, pos0, DEV, pad_rows_to=8)
    torch.manual_seed(7)
    qw, kw = H * hd, Hk * hd
    qkv = torch.randn(lay.n_rows, qw + 2 * kw, device=DEV).to(torch.bfloat16)
    r = 0
    for s, n in enumerate(new):                            # the step's own keys and values
        qkv[r:r + n, qw:qw + kw] = dk[s][pos0[s]:].reshape(n, kw).to(DEV)
        qkv[r:r + n, qw + kw:] = dv[s][pos0[s]:].reshape(n, kw).to(DEV)
        r += n
    out = torch.full((lay.n_rows, qw), 7.0, device=DEV, dtype=torch.bfloat16)
    scale = 0.6 / math.sqrt(hd)
    launches = ops.launches
    ops.attention(qkv, 0, lay, kv, H, out, scale, window, (qw, qw + kw))
    assert ops.launches == launches + 1                    # no pass of its own for the append
    ops.check_device_errors()
    r = 0
    for s, n in enumerate(new):
        q = qkv[r:r + n, :qw].view(n, H, hd).double().cpu()
        k, v = dk[s].double(), dv[s].double()
        qpos = torch.arange(pos0[s], pos0[s] + n)[:, None]
        key = torch.arange(lens[s])[None, :]
        vis = key <= qpos
        if window > 0:
            vis &= key > qpos - window
        for h in range(H):
            sc = (q[:, h] @ k[:, h // (H // Hk)].t()) * scale
            ref = torch.softmax(sc.masked_fill(~vis, float("-inf")), dim=1) @ v[:, h // (H // Hk)]
            got = out[r:r + n, h * hd:(h + 1) * hd].double().cpu()
            err = (got - ref).abs().max(dim=1).values
            assert err.max() <= 1.5e-2 * max(1.0, float(ref.abs().max())), \
                f"sequence {s}, head {h}, worst row {int(err.argmax())}"
        # every token of the sequence is in the cache now, bit for bit
        for pos in range(lens[s]):
            page = int(table[s + 1, pos // PAGE])
            assert torch.equal(kv.k[page, :, pos % PAGE], kv_true.k[page, :, pos % PAGE]), (s, pos)
            assert torch.equal(kv.v[page, :, pos % PAGE], kv_true.v[page, :, pos % PAGE]), (s, pos)
        r += n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_far_key_among_hundreds_is_found(ops, dtype):
    """One key, hundreds of positions back and on another page, is made to dominate."""
    H, hd, L = 2, 64, 700
    kv, dk, dv = _paged_cache(1, [L], H, hd, dtype, seed=9)
    lay = build_layout([(1, [0], [])], [L - 1], DEV)
    q = torch.randn(1, 3 * H * hd).to(dtype)
    far = 37
    for h in range(H):
        q[0, h * hd:(h + 1) * hd] = (dk[0][far, h].float() * 3.0).to(dtype)   # score stands out
    out = torch.empty(1, H * hd, device=DEV, dtype=dtype)
    ops.attention(q.to(DEV), 0, lay, kv, H, out, 1.0, 0)
    ref = _attention_ref(q[0, :H * hd].view(H, hd), dk[0], dv[0], L - 1, 1.0, 1)
    assert (ref - dv[0][far].double()).abs().max() < 1e-3          # the far value is the answer
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    assert (out.view(H, hd).double().cpu() - ref).abs().max() <= tol * float(ref.abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd", [32, 12])                 # 16-byte pieces / single elements
def test_kv_append_writes_only_its_rows(ops, dtype, hd):
    Hk = 3
    lens = [130, 5, 200]
    kv, dk, dv = _paged_cache(3, lens, Hk, hd, dtype, seed=2)
    k_before, v_before = kv.k.clone(), kv.v.clone()
    # positions 127..129 (two pages), 0..4, and 50..199 (three pages)
    entries = [(1, [0] * 3, []), (2, [0] * 5, []), (3, [0] * 150, [])]
    lay = build_layout(entries, [127, 0, 50], DEV, pad_rows_to=16)
    width = 5 * hd + 2 * Hk * hd
    src = torch.randn(lay.n_rows, width, device=DEV).to(dtype)
    ops.kv_append(src, 5 * hd, 5 * hd + Hk * hd, lay.row_slot, lay.row_pos, kv, lay.n_rows)
    expect_k, expect_v = k_before.clone(), v_before.clone()
    r = 0
    table = kv.block_table.cpu()
    for slot, pos0, n in ((1, 127, 3), (2, 0, 5), (3, 50, 150)):
        for i in range(n):
            pos = pos0 + i
            page = int(table[slot, pos // PAGE])
            expect_k[page, :, pos % PAGE] = src[r, 5 * hd:5 * hd + Hk * hd].view(Hk, hd)
            expect_v[page, :, pos % PAGE] = src[r, 5 * hd + Hk * hd:].view(Hk, hd)
            r += 1
    assert torch.equal(kv.k, expect_k) and torch.equal(kv.v, expect_v)


@pytest.mark.parametrize("vocab, n_keep", [(50257, 1024), (513, 64), (40, 64), (3000, 1)])
def test_the_largest_logits_of_a_row(ops, vocab, n_keep):
    """The candidates kernel: every element not smaller than the n_keep-th largest, the row
    maximum and the f64 softmax denominator; ties at the threshold; a NaN row; fewer elements
    than asked for."""
    torch.manual_seed(vocab)
    logits = torch.randn(5, vocab, device=DEV) * 3.0
    logits[1, :7] = logits[1].max()                                  # ties at the top
    if vocab > n_keep + 40:
        thr = logits[2].sort(descending=True).values[n_keep - 1]
        logits[2, logits[2].argsort()[:50]] = thr                    # 50 more ties at the threshold
    logits[3, 5] = float("nan")
    logits[4, 1::2] = float("-inf")
    temp = 0.7
    keep = min(n_keep, vocab)
    vals, idx, counts, stats = ops.top_candidates(logits, keep, temp)
    vals, idx, counts, stats = vals.cpu(), idx.cpu(), counts.cpu(), stats.cpu()
    cap = vals.shape[1]
    for r in range(5):
        row = logits[r].cpu()
        if r == 3:
            assert counts[r] == -1
            continue
        thr = row.sort(descending=True).values[keep - 1]
        want = set(torch.nonzero(row >= thr).flatten().tolist())
        assert counts[r] == len(want)
        if len(want) <= cap:
            got = idx[r, :counts[r]].tolist()
            assert set(got) == want and len(got) == len(want)
            assert torch.equal(vals[r, :counts[r]], row[idx[r, :counts[r]].long()])
        else:
            assert r == 2
        assert stats[r, 0] == row.max().double()
        ref = torch.exp(row.double() / temp - row.max().double() / temp).sum()
        assert abs(stats[r, 1] - ref) <= 1e-12 * ref


def test_argmax_first_maximum(ops):
    torch.manual_seed(3)
    logits = torch.randn(9, 50257, device=DEV)
    logits[0, 77] = logits[0, 40000] = 50.0          # a tie: the lower index wins
    logits[1, 0] = 60.0
    logits[2, 50256] = 60.0
    logits[3, 5] = float("nan")
    logits[4] = -float("inf")
    logits[5, 0] = float("nan")                      # the scan starts from a NaN and stays there
    out = torch.empty(9, device=DEV, dtype=torch.int32)
    ops.argmax(logits, out)
    got = out.cpu().tolist()
    assert got[0] == 77 and got[1] == 0 and got[2] == 50256 and got[4] == 0 and got[5] == 0
    row3 = logits[3].cpu()
    row3[5] = -float("inf")
    assert got[3] == int(torch.argmax(row3))
    assert got[6:] == torch.argmax(logits[6:], dim=-1).cpu().tolist()
    small = torch.tensor([[0.1, 5.0, 5.0, -1.0]], device=DEV)     # src/sampler.rs:223-228
    o = torch.empty(1, device=DEV, dtype=torch.int32)
    ops.argmax(small, o)
    assert int(o) == 1


def test_temperature_sampling_matches_the_host_sampler(ops):
    from nimbus_infer_rs_b200.sampling import SamplingParams, Xoshiro256pp
    from nimbus_infer_rs_b200.sampling import host as H
    torch.manual_seed(4)
    V, n = 1000, 64
    logits = torch.randn(n, V, device=DEV) * 3
    for temp in (0.7, 1.0, 1e-9):
        rngs = [Xoshiro256pp(100 + i) for i in range(n)]
        u = torch.tensor([r.next_f64() for r in rngs], dtype=torch.float64, device=DEV)
        out = torch.empty(n, device=DEV, dtype=torch.int32)
        ops.sample_temperature(logits, temp, u, out)
        rngs = [Xoshiro256pp(100 + i) for i in range(n)]
        want = [H.sample(logits[i].cpu().numpy(), SamplingParams(temperature=temp), [], rngs[i])
                for i in range(n)]
        assert out.cpu().tolist() == want
    # edges of the cumulative sum
    two = torch.tensor([[0.0, 0.0, -float("inf")]], device=DEV)
    o = torch.empty(1, device=DEV, dtype=torch.int32)
    for uu, w in ((0.0, 0), (0.49, 0), (0.51, 1), (0.999999, 1)):
        ops.sample_temperature(two, 1.0, torch.tensor([uu], dtype=torch.float64, device=DEV), o)
        assert int(o) == w
    ops.sample_temperature(torch.full((1, 7), -float("inf"), device=DEV), 1.0,
                           torch.tensor([0.3], dtype=torch.float64, device=DEV), o)
    assert int(o) == 0


@pytest.mark.parametrize("V, k", [(1000, 1), (1000, 40), (777, 776), (777, 777), (513, 5000),
                                  (50257, 50), (4099, 2000)])
def test_top_k_sampling_matches_the_host_sampler(ops, V, k):
    """Top-k sampling on the device against the float64 sampler of the host, draw for draw:
    ties at the k-th value, rows with -inf entries, k at and beyond the vocabulary, tiny and
    large temperatures; a row with a NaN is handed back (-1)."""
    from nimbus_infer_rs_b200.sampling import SamplingParams, Xoshiro256pp
    from nimbus_infer_rs_b200.sampling import host as H
    torch.manual_seed(V + k)
    n = 24
    logits = torch.randn(n, V, device=DEV) * 3
    logits[1, 5:25] = logits[1].max()                       # ties at the top
    kth = logits[2].topk(min(k, V)).values[-1]
    logits[2, :7] = kth                                     # ties at the threshold
    logits[3, ::3] = -float("inf")
    logits[4] = torch.round(logits[4])                      # many equal values
    logits[5, 10] = 0.0
    logits[5, 11] = -0.0
    for temp in (0.7, 1.0, 1e-9, 30.0):
        rngs = [Xoshiro256pp(7 + i) for i in range(n)]
        u = torch.tensor([r.next_f64() for r in rngs], dtype=torch.float64, device=DEV)
        out = torch.empty(n, device=DEV, dtype=torch.int32)
        ops.sample_top_k(logits, k, temp, u, out)
        rngs = [Xoshiro256pp(7 + i) for i in range(n)]
        p = SamplingParams(temperature=temp, top_k=k)
        want = [H.sample(logits[i].cpu().numpy(), p, [], rngs[i]) for i in range(n)]
        assert out.cpu().tolist() == want, temp
    bad = logits[:2].clone()
    bad[1, 3] = float("nan")
    out = torch.empty(2, device=DEV, dtype=torch.int32)
    ops.sample_top_k(bad, k, 1.0, torch.tensor([0.5, 0.5], dtype=torch.float64, device=DEV), out)
    assert int(out[1]) == -1 and int(out[0]) >= 0
    ops.sample_top_k(torch.full((1, 9), -float("inf"), device=DEV), k, 1.0,
                     torch.tensor([0.3], dtype=torch.float64, device=DEV), out[:1])
    assert int(out[0]) == 0


@pytest.mark.parametrize("V, k, top_p", [(1000, 0, 0.9), (1000, 40, 0.5), (777, 0, 0.0), (513, 0, 0.3),
                                         (50257, 0, 0.9), (50257, 1024, 0.95), (4099, 7, 0.999),
                                         (300, 299, 0.7), (50257, 0, 0.5)])
def test_top_p_sampling_matches_the_host_sampler(ops, V, k, top_p):
    """Top-p (and top-k with it) on the device against the float64 sampler of the host, draw for
    draw: peaked rows (the cut among the first few tokens), ties across the cut, rows with -inf,
    a flat row (handed back: -2, unless the vocabulary is small enough to be listed whole) and a
    row with a NaN (-1)."""
    from nimbus_infer_rs_b200.sampling import SamplingParams, Xoshiro256pp
    from nimbus_infer_rs_b200.sampling import host as H
    torch.manual_seed(V + k)
    n = 24
    logits = torch.randn(n, V, device=DEV) * 4
    logits[1, 5:25] = logits[1].max()                       # ties at the top, across the cut
    logits[2, 100:103] = logits[2].max() + 6.0              # three tokens hold nearly all the mass
    logits[3, ::3] = -float("inf")
    logits[4] = torch.round(logits[4])                      # many equal values
    logits[5] = logits[5] * 0.001                           # flat
    logits[6, 7] = logits[6].max() + 30.0                   # one token alone
    handed_back = 0
    for temp in (0.7, 1.0, 2.5):
        rngs = [Xoshiro256pp(7 + i) for i in range(n)]
        u = torch.tensor([r.next_f64() for r in rngs], dtype=torch.float64, device=DEV)
        out = torch.empty(n, device=DEV, dtype=torch.int32)
        ops.sample_top_p(logits, k, top_p, temp, u, out)
        got = out.cpu().tolist()
        rngs = [Xoshiro256pp(7 + i) for i in range(n)]
        p = SamplingParams(temperature=temp, top_k=k, top_p=top_p)
        for i in range(n):
            want = H.sample(logits[i].cpu().numpy(), p, [], rngs[i])
            if got[i] == -2:
                handed_back += 1
                continue
            assert got[i] == want, (temp, i)
    assert handed_back <= 3 * n // 2                        # most rows are settled on the device
    if V <= 1024 or (0 < k <= 1024):
        assert handed_back == 0                             # the universe is listed whole
    bad = logits[:2].clone()
    bad[1, 3] = float("nan")
    out = torch.empty(2, device=DEV, dtype=torch.int32)
    ops.sample_top_p(bad, k, top_p, 1.0, torch.tensor([0.5, 0.5], dtype=torch.float64, device=DEV), out)
    assert int(out[1]) == -1 and int(out[0]) != -1


def test_repetition_penalty(ops):
    logits = torch.tensor([[2.0, -2.0, 1.0, 3.0], [1.0, 1.0, 1.0, 1.0]], device=DEV)
    hist = torch.tensor([[0, 1, 1, 0], [3, -1, -1, -1]], device=DEV, dtype=torch.int32)
    lens = torch.tensor([4, 1], device=DEV, dtype=torch.int32)
    ops.repetition_penalty(logits, hist, lens, 2.0)
    assert logits.cpu().tolist() == [[1.0, -4.0, 1.0, 3.0], [1.0, 1.0, 1.0, 0.5]]


@pytest.mark.parametrize("M, N, K", [(1, 64, 64), (8, 2304, 768), (17, 100, 96), (64, 768, 3072),
                                     (40, 1001, 1600), (3, 77, 100), (130, 257, 72),
                                     (8, 520, 3072), (16, 96, 4096), (2, 72, 8192), (11, 264, 1600)])
@pytest.mark.parametrize("wdt", [torch.float32, torch.bfloat16])
def test_linear_with_norm_of_the_rows_first(ops, M, N, K, wdt):
    """LayerNorm fused into the product (few rows) or run before it (many rows) must both
    equal norm-then-product in float64, up to the rounding of the normalised rows."""
    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device=DEV) * 2 + 0.3
    gamma, beta = torch.randn(K, device=DEV), torch.randn(K, device=DEV)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(wdt)
    bias = torch.randn(N, device=DEV)
    act_dtype = wdt
    xd = x.double()
    mean = xd.mean(-1, keepdim=True)
    h = (xd - mean) / torch.sqrt(((xd - mean) ** 2).mean(-1, keepdim=True) + 1e-5) * gamma.double() \
        + beta.double()
    ref = _gelu(h @ w.double().t() + bias.double(), 1)
    out = torch.empty(M, N, device=DEV, dtype=torch.float32)
    ops.linear(x, w, bias, out, 1, None, (gamma, beta, 1e-5, act_dtype))
    tol = (2e-5 if wdt == torch.float32 else 1.5e-2) * float(ref.abs().max())
    assert (out.double() - ref).abs().max() <= tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, Hk, hd, window", [(12, 12, 64, 0), (4, 4, 16, 0), (6, 2, 32, 0),
                                               (8, 1, 128, 0), (6, 2, 64, 100), (3, 3, 48, 0),
                                               (25, 25, 64, 0), (16, 1, 64, 0)])
@pytest.mark.parametrize("max_kv", [64, 1024, 4096])
@pytest.mark.parametrize("clusters", [True, False])
def test_decode_attention_over_splits(ops, dtype, H, Hk, hd, window, max_kv, clusters):
    """One query row per sequence (a decode step): sequences of very unequal lengths, pages
    shuffled, a padding row in the middle; run twice on the same scratch (the counters must be
    left at zero).  `max_kv` (the longest context the launch is sized for) changes the number
    of splits a sequence's pages are spread over.  The splits of the bfloat16 kernel merge in
    the shared memory of a thread-block cluster (at most 8 of them) or, with `clusters` off,
    through scratch memory and a counter like the 32-bit kernel's."""
    if dtype == torch.float32 and not clusters:
        pytest.skip("the 32-bit kernel has one way to merge")
    was = ops.decode_clusters
    ops.set_decode_clusters(clusters)
    try:
        _decode_attention_over_splits(ops, dtype, H, Hk, hd, window, max_kv)
    finally:
        ops.set_decode_clusters(was)


def _decode_attention_over_splits(ops, dtype, H, Hk, hd, window, max_kv):
    lens = [1, 64, 65, 700, 333, 1000, 129]
    kv, dk, dv = _paged_cache(len(lens), lens, Hk, hd, dtype, seed=H + hd)
    entries = [(s + 1, [0], []) for s in range(len(lens))]
    lay = build_layout(entries, [l - 1 for l in lens], DEV, pad_rows_to=8)
    assert lay.is_decode
    lay.max_kv_len = max_kv if max_kv >= max(lens) else max(lens)
    # a padding row between live rows
    lay.row_slot[2] = -1
    torch.manual_seed(6)
    qkv = torch.randn(lay.n_rows, (H + 2 * Hk) * hd, device=DEV).to(dtype)
    scale = 0.5 / math.sqrt(hd)
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    for attempt in range(2):
        out = torch.full((lay.n_rows, H * hd), 7.0, device=DEV, dtype=dtype)
        ops.attention(qkv, 0, lay, kv, H, out, scale, window)
        for s, l in enumerate(lens):
            if s == 2:
                assert (out[s] == 0).all()
                continue
            ref = _attention_ref(qkv[s, :H * hd].view(H, hd).cpu(), dk[s], dv[s], l - 1, scale,
                                 H // Hk, window)
            got = out[s].view(H, hd).double().cpu()
            assert (got - ref).abs().max() <= tol * max(1.0, float(ref.abs().max())), (attempt, s)
        assert (out[len(lens):] == 0).all()


@pytest.mark.parametrize("M, N, K", [(65, 64, 8), (128, 128, 64), (129, 200, 72), (300, 2304, 768),
                                     (2048, 768, 3072), (1000, 3072, 768), (256, 50257, 768),
                                     (2048, 96, 320), (4096, 4096, 1600), (77, 1001, 2000),
                                     (2048, 1536, 256), (640, 800, 128),
                                     (64, 768, 3072), (100, 2304, 768), (17, 776, 520),
                                     (2048, 2304, 768), (700, 1000, 256),
                                     (40, 520, 1600), (96, 136, 6400)])
@pytest.mark.parametrize("pairs", [False, True])
def test_tensor_core_product(ops, M, N, K, pairs):
    """The tcgen05 kernel (bf16, more than 64 rows) against float64: tile edges in M, N and K,
    all tile widths (64, 96, 128, 192, 256), every epilogue, products of at most 128 rows (one
    row tile), K cut among a cluster of CTAs (few rows, long K), pairs of CTAs; and no wait may have timed out."""
    if pairs and M <= 128:
        pytest.skip("pairs of CTAs take products of more than 128 rows")
    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    bias = torch.randn(N, device=DEV)
    ref0 = x.double() @ w.double().t()
    tol = 3e-6 * float(ref0.abs().max()) * math.sqrt(K / 64)
    out = torch.empty(M, N, device=DEV)
    ops.set_pairs(2 if pairs else 0)       # 256-row tiles on pairs of CTAs (cta_group::2)
    try:
        _check_tensor_core_product(ops, x, w, bias, ref0, tol, out, M, N)
    finally:
        ops.set_pairs(1)


def _check_tensor_core_product(ops, x, w, bias, ref0, tol, out, M, N):
    ops.linear(x, w, None, out)
    err = (out.double() - ref0).abs()
    assert err.max() <= tol, f"worst element {err.argmax().item() // N, err.argmax().item() % N}"
    ref = _gelu(ref0 + bias.double(), 1)
    o = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    ops.linear(x, w, bias, o, 1)
    assert (o.double() - ref).abs().max() <= tol + 8e-3 * float(ref.abs().max())
    res = torch.randn(M, N, device=DEV)
    stream = res.clone()
    ops.linear(x, w, bias, stream, 0, stream)
    ref = ref0 + bias.double() + res.double()
    assert (stream.double() - ref).abs().max() <= tol + 1e-6 * float(ref.abs().max())
    ops.check_device_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, Hk, hd", [(12, 12, 64), (6, 2, 32), (4, 1, 128), (4, 4, 16)])
@pytest.mark.parametrize("max_kv", [512, 4096])
def test_decode_attention_appends_its_own_key_and_value(ops, dtype, H, Hk, hd, max_kv):
    """With `append`, the decode kernel must give what append-then-attend gives, and leave the
    same cache behind; positions at a page start, a page end and mid-page."""
    lens = [1, 64, 65, 128, 300, 449]               # the new token is the last of each
    kv_a, dk, dv = _paged_cache(len(lens), lens, Hk, hd, dtype, seed=3 * H + hd)
    kv_b = LayerKV(kv_a.k.clone(), kv_a.v.clone(), kv_a.block_table, PAGE, Hk, hd)
    lay = build_layout([(s + 1, [0], []) for s in range(len(lens))], [l - 1 for l in lens], DEV)
    lay.max_kv_len = max_kv
    torch.manual_seed(8)
    qkv = torch.randn(lay.n_rows, (H + 2 * Hk) * hd, device=DEV).to(dtype)
    kc, vc = H * hd, (H + Hk) * hd
    want = torch.empty(lay.n_rows, H * hd, device=DEV, dtype=dtype)
    ops.kv_append(qkv, kc, vc, lay.row_slot, lay.row_pos, kv_a, lay.n_rows)
    ops.attention(qkv, 0, lay, kv_a, H, want, 0.2)
    got = torch.empty_like(want)
    ops.attention(qkv, 0, lay, kv_b, H, got, 0.2, 0, (kc, vc))
    assert torch.equal(kv_a.k, kv_b.k) and torch.equal(kv_a.v, kv_b.v)
    assert torch.equal(got, want)


def test_a_wait_that_runs_out_is_reported_and_the_next_product_is_right(ops):
    """Every wait on a barrier in the tensor-core kernels has a clock budget; a wait that runs
    out makes the kernel give up, free what it holds, return, and raise a word in pinned host
    memory that the host reads where it waits for results anyway.  The probe runs that same
    bounded wait on a barrier that nothing ever completes.  Then a real product runs with a
    budget of zero cycles: each of its waits either finds its barrier complete already or
    gives up at once, so the kernel either finishes with the right result or returns early and
    says so; never a wrong result without the word.  With the budget restored the same
    product is right and nothing is reported."""
    from nimbus_infer_rs_b200.csrc.ops import KernelError
    ops.check_device_errors()                               # nothing pending from earlier tests
    torch.manual_seed(3)
    M, N, K = 128, 192, 2048
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV) * 0.05).to(torch.bfloat16)
    ref = x.double() @ w.double().t()
    tol = 1e-2 * float(ref.abs().max())
    try:
        ops.set_wait_budget(20_000)                         # about ten microseconds
        assert ops.wait_probe() == 2                        # gave up after the budget
        with pytest.raises(KernelError, match="wait_probe"):
            ops.raise_device_errors()
        ops.raise_device_errors()                           # reading lowered the word
        ops.set_wait_budget(0)
        out = torch.zeros(M, N, device=DEV)
        ops.linear(x, w, None, out)
        try:
            ops.check_device_errors()
            gave_up = False
        except KernelError as e:
            gave_up = True
            assert "gemm_tcgen05" in str(e)
        if not gave_up:
            assert (out.double() - ref).abs().max() <= tol
    finally:
        ops.set_wait_budget(None)
    out = torch.zeros(M, N, device=DEV)
    ops.linear(x, w, None, out)
    ops.check_device_errors()
    assert (out.double() - ref).abs().max() <= tol


STREAM_SHAPES = [  # M, N, K, norm first?
    (8, 2304, 768, True), (8, 768, 768, False), (8, 3072, 768, True), (8, 768, 3072, False),
    (8, 50257, 768, True), (1, 50257, 768, True), (1, 768, 3072, False), (16, 4800, 1600, True),
    (9, 1600, 6400, False), (16, 1600, 6400, False), (5, 777, 80, True), (7, 80, 136, False),
    (3, 1000, 96, True), (2, 72, 8192, True), (13, 264, 1600, True), (4, 50257, 1600, True),
    (12, 4104, 1024, True), (6, 8, 8, False)]


@pytest.mark.parametrize("M, N, K, ln", STREAM_SHAPES)
def test_products_of_a_decode_step(ops, M, N, K, ln):
    """At most 16 rows, bf16 weights: the kernel that brings its weight rows into shared memory
    before it waits for its predecessor.  One batch of columns per CTA (a layer's products), a
    long walk through the ring (the head's 50,257 columns), K cut into chunks when a stage
    cannot hold whole rows, rows 9..16, widths that are no multiple of 32 and outputs that are
    no multiple of 8; with the norm of the rows folded in, bias, GELU, the residual added in
    place, bf16 and fp32 results: all against float64."""
    taken = bool(ops.lib.nb_gemm_stream_supported(M, N, K, 0))
    assert ops.use_stream and (taken or K >= 6400)         # very long rows go to the other kernel
    torch.manual_seed(M + N + K)
    w = (torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    bias = torch.randn(N, device=DEV)
    if ln:
        x = torch.randn(M, K, device=DEV) * 2 + 0.3
        gamma, beta = torch.randn(K, device=DEV), torch.randn(K, device=DEV)
        xd = x.double()
        mean = xd.mean(-1, keepdim=True)
        h = (xd - mean) / torch.sqrt(((xd - mean) ** 2).mean(-1, keepdim=True) + 1e-5) \
            * gamma.double() + beta.double()
        norm = (gamma, beta, 1e-5, torch.bfloat16)
        xin = x
    else:
        xin = torch.randn(M, K, device=DEV).to(torch.bfloat16)
        h, norm = xin.double(), None
    pre = h @ w.double().t() + bias.double()
    before = ops.launches
    # GELU, bf16 result
    ref = _gelu(pre, 1)
    out = torch.full((M, N), 9.0, device=DEV, dtype=torch.bfloat16)
    ops.linear(xin, w, bias, out, 1, None, norm)
    tol = 1.5e-2 * float(ref.abs().max())
    assert (out.double() - ref).abs().max() <= tol
    # residual added in place on the fp32 stream, no bias
    res = torch.randn(M, N, device=DEV)
    ref = (h @ w.double().t()) + res.double()
    stream = res.clone()
    ops.linear(xin, w, None, stream, 0, stream, norm)
    assert (stream.double() - ref).abs().max() <= 1.5e-2 * float(ref.abs().max())
    fused = (not ln) or ops.lib.nb_gemm_stream_supported(M, N, K, 1)
    if taken:
        assert ops.launches - before == (2 if fused else 4)     # a norm that cannot be folded in runs first
    # the other kernel for few rows gives the same within rounding
    ops.use_stream = False
    try:
        other = res.clone()
        ops.linear(xin, w, None, other, 0, other, norm)
    finally:
        ops.use_stream = True
    assert (other.double() - stream.double()).abs().max() <= 1.5e-2 * float(ref.abs().max())
    ops.check_device_errors()
