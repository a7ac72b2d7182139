"""How the launchers cut a product, and which shapes they take or refuse: host code of the kernel
library, called without a GPU.  A wrong plan does not show as a wrong number in a test on the
GPU but as a kernel that waits for a block of K that never comes, so the arithmetic is pinned
here, over many more shapes than the GPU tests launch."""
import ctypes
import itertools

import pytest

from nimbus_infer_rs_b200.csrc import build


@pytest.fixture(scope="module")
def lib():
    try:
        return build.load()
    except build.BuildError as e:              # no compiler and no built library on this machine
        pytest.skip(str(e))


SMEM_MAX = 227 * 1024


def test_few_rows_tensor_core_product_plans(lib):
    """gemm_tc_rows.cu:plan_rows.  Every CTA of a cluster has a block of K, the CTAs' shares of
    the rows cover all rows, the receive buffer's row pitch is an odd number of 16-byte units,
    the ring fits."""
    out = (ctypes.c_int * 6)()
    taken = 0
    for M, N, K in itertools.product((1, 16, 17, 31, 33, 64, 96, 100, 128),
                                     (8, 120, 768, 1600, 2304, 4736, 6400, 18944),
                                     (8, 64, 72, 768, 1536, 1600, 3072, 6400, 8192)):
        for force in (0, 1, 2, 3, 5, 8):
            lib.nb_gemm_tc_rows_force_split(force)
            ok = lib.nb_gemm_tc_rows_plan(M, N, K, out)
            lib.nb_gemm_tc_rows_force_split(0)
            assert ok == lib.nb_gemm_tc_rows_supported(M, N, K) or force
            if not ok:
                continue
            taken += 1
            nb, split, kb_per, stages, chunk, smem = list(out)
            num_kb = (K + 63) // 64
            assert nb % 16 == 0 and M <= nb < M + 16
            assert 1 <= split <= 8 and (force in (0, split))
            assert split * kb_per >= num_kb                       # every block of K has a CTA
            assert (split - 1) * kb_per < num_kb                  # and every CTA a block
            assert chunk % 4 == 0 and chunk * split >= nb
            assert 1 <= stages <= min(8, kb_per)
            assert smem <= SMEM_MAX
            assert (N + 127) // 128 * split <= 148 or split == 1
    assert taken > 1000
    # refused, not mangled
    for M, N, K in ((0, 768, 768), (129, 768, 768), (64, 768, 4), (64, 768, 100), (64, 0, 768),
                    (64, 50257, 768)):
        assert lib.nb_gemm_tc_rows_supported(M, N, K) == 0
        assert lib.nb_gemm_tc_rows_preferred(M, N, K) == 0


def test_where_the_few_rows_product_is_preferred(lib):
    """A long K over few columns (measured): the MLP's second product of GPT-2 small at 32 to
    96 rows, XL's at up to 128 rows; not the products over K = 768."""
    pref = lib.nb_gemm_tc_rows_preferred
    assert pref(64, 768, 3072) and pref(32, 768, 3072) and pref(96, 768, 3072)
    assert pref(128, 1600, 6400) and pref(64, 1600, 1600)
    assert pref(96, 768, 1536) and not pref(128, 768, 1536)   # 128 rows: K of 48 blocks and more
    assert pref(128, 768, 3072)
    assert not pref(64, 2304, 768) and not pref(64, 3072, 768) and not pref(64, 768, 768)
    assert not pref(64, 6400, 1600)            # too many columns: the tiled kernel fills the GPU


def test_weight_streaming_product_plans(lib):
    """gemm_stream.cuh:plan_stream.  At most 16 rows; the work items of a batch of column
    groups cover K; the CTAs fit the GPU and their shared memory an SM."""
    out = (ctypes.c_int * 13)()
    taken = 0
    for M, N, K, ln in itertools.product((1, 2, 7, 8, 9, 16), (8, 120, 768, 2304, 6400, 50257),
                                         (64, 120, 768, 1600, 3072, 6400), (0, 1)):
        ok = lib.nb_gemm_stream_plan(M, N, K, ln, out)
        assert ok == lib.nb_gemm_stream_supported(M, N, K, ln)
        if not ok:
            continue
        taken += 1
        gb, wn, k_item, n_kc, stages, pitch, x_stride, tpr, n16, nw, vpt, grid, smem = list(out)
        assert k_item % 64 == 0 and k_item * n_kc >= K            # the items cover K
        assert k_item * (n_kc - 1) < K                            # and none is empty
        assert n16 == (N + 15) // 16
        assert 1 <= grid and 1 <= stages and gb >= 1 and wn >= 1
        assert nw * 32 <= 1024 and smem <= SMEM_MAX
        assert x_stride >= K
    assert taken > 100
    assert lib.nb_gemm_stream_supported(17, 768, 768, 0) == 0     # more than 16 rows
    assert lib.nb_gemm_stream_supported(0, 768, 768, 0) == 0


def test_which_attention_shapes_the_decode_kernel_takes(lib):
    """attention_decode.cu: bfloat16 head sizes in steps of 16 up to 128, any number of heads in
    groups of up to 8 query heads a key head, pages of 64 tokens; everything else is refused
    (the caller then uses the kernel for any shape)."""
    sup = lib.nb_attention_decode_supported
    import torch
    from nimbus_infer_rs_b200.csrc import ops
    BF16, F32 = ops._DTYPE_CODE[torch.bfloat16], ops._DTYPE_CODE[torch.float32]
    for hd in range(8, 160, 8):
        assert sup(BF16, hd, 12, 12, 64) == int(hd % 16 == 0 and hd <= 128)
        assert sup(F32, hd, 12, 12, 64) == int(hd in (16, 32, 64, 128))
    for heads, kv in ((1, 1), (25, 25), (7, 7), (6, 3), (12, 4), (16, 2), (5, 1)):
        assert sup(BF16, 64, heads, kv, 64) == 1
    assert sup(BF16, 64, 12, 5, 64) == 0           # heads not a multiple of key heads
    assert sup(BF16, 64, 18, 2, 64) == 0           # groups of 9
    assert sup(BF16, 64, 12, 12, 32) == 0 and sup(BF16, 64, 12, 12, 128) == 0   # other pages
    acc, ml, cn = ctypes.c_longlong(), ctypes.c_longlong(), ctypes.c_longlong()
    lib.nb_attention_decode_scratch(8, 12, 4, 64, 5, ctypes.byref(acc), ctypes.byref(ml),
                                    ctypes.byref(cn))
    assert (acc.value, ml.value, cn.value) == (8 * 12 * 5 * 64, 8 * 12 * 5 * 2, 8 * 4)


def test_which_shapes_the_other_kernels_take(lib):
    """The prefill attentions and the products say which shapes are theirs; what none of the fast
    kernels takes goes to the kernels for any shape (attention_generic.cu, gemm_simt.cu), so a
    configuration is never run by a kernel that was not written for it."""
    import torch
    from nimbus_infer_rs_b200.csrc import ops
    BF16, F32 = ops._DTYPE_CODE[torch.bfloat16], ops._DTYPE_CODE[torch.float32]
    tc, mma, f32 = (lib.nb_attention_prefill_tc_supported, lib.nb_attention_prefill_supported,
                    lib.nb_attention_prefill_f32_supported)
    for hd in range(16, 144, 16):
        d = 12 * hd
        assert tc(BF16, hd, 12, 12, 64, 3 * d, 0, BF16, d) == int(hd in (64, 128))
        assert mma(BF16, hd, 12, 12, 64, 3 * d, 0) == int(hd in (16, 32, 48, 64, 96, 128))
        assert f32(hd, 12, 12, 64) == int(hd in (64, 128))
    assert tc(F32, 64, 12, 12, 64, 2304, 0, F32, 768) == 0          # a 32-bit run
    assert tc(BF16, 64, 12, 12, 32, 2304, 0, BF16, 768) == 0        # another page size
    assert tc(BF16, 64, 12, 5, 64, 2304, 0, BF16, 768) == 0         # heads and key heads
    assert tc(BF16, 64, 12, 12, 64, 2300, 0, BF16, 768) == 0        # a row pitch TMA cannot take
    assert tc(BF16, 64, 12, 12, 64, 2304, 4, BF16, 768) == 0        # a first column it cannot take
    assert tc(BF16, 64, 12, 12, 64, 2304, 0, BF16, 772) == 0        # 16-byte stores of the result
    assert tc(BF16, 64, 12, 12, 64, 2304, 0, F32, 772) == 1
    assert mma(BF16, 64, 12, 12, 64, 2300, 0) == 0 and mma(F32, 64, 12, 12, 64, 2304, 0) == 0

    gemm = lib.nb_gemm_tcgen05_supported
    assert gemm(BF16, BF16, 2048, 768, 768) and gemm(BF16, BF16, 1, 8, 8)
    assert gemm(BF16, BF16, 130, 50257, 1600)                        # a width that is no power of two
    assert not gemm(BF16, BF16, 64, 768, 100)                        # rows of K that TMA cannot take
    assert not gemm(F32, BF16, 64, 768, 768) and not gemm(BF16, F32, 64, 768, 768)
    assert not gemm(BF16, BF16, 0, 768, 768)

    norm = lib.nb_gemm_skinny_norm_supported
    assert norm(8, 2304, 768) and norm(16, 4800, 1600) and norm(1, 50257, 768)
    assert not norm(17, 2304, 768) and not norm(8, 2304, 100) and not norm(8, 2304, 1 << 16)
