"""Tensor-level face of the kernel library.

Each function checks its tensors and hands raw pointers plus the current CUDA stream to one
``extern "C"`` launcher of ``libnimbus_b200.so``.  There is no other implementation in the
package: if the library cannot be built or loaded, the first call raises.

The functions go through a backend object so that a test can drive the engine's host logic
(batching, paging, slots) with a stand-in of its own; the package itself only ever
installs :class:`CudaBackend`.
"""
from __future__ import annotations

import os

import torch

ACT_NONE, ACT_GELU_TANH, ACT_GELU_ERF = 0, 1, 2
ACTIVATIONS = {"none": ACT_NONE, "gelu_tanh": ACT_GELU_TANH, "gelu_erf": ACT_GELU_ERF}

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
DECODE_TARGET_CTAS = 4 * 148   # CTAs the split 32-bit decode attention aims to put on the GPU
# CTAs the tensor-core prefill attention aims to put on the GPU by cutting the keys of a tile
# into runs: one per SM.  (Two of its CTAs on an SM are bound by instruction issue, so cutting
# further only adds the merge; measured on GPT-2 124M, 2 x 1024 tokens.)
PREFILL_TARGET_CTAS = 148
FUSED_NORM_MAX_ROWS = 16       # a LayerNorm is folded into the product up to this many rows
FUSED_NORM_MAX_COLS = 16384    # ... and output columns (a long weight stream wants the leaner kernel)
SKINNY_MAX_ROWS = 64   # matrix products with at most this many rows take the weight-streaming kernel
STREAM_MAX_ROWS = 16   # ... and with at most this many the kernel that stages weights in shared memory
ROWS_MAX_ROWS = 128    # up to this many rows a product's weights are the tensor cores' 128-row operand


def decode_splits(base_ctas: int, pages: int, page: int, head_dim: int, sms: int, most: int) -> int:
    """Splits of a sequence's pages in the tensor-core decode attention (swept on a B200 at
    contexts of 256 and 1,024 and batches of 1 to 32).  Four pages a split: eight warps take
    two at a time, so a split is two turns of the loop and every page is asked for before the
    kernel's wait.  Fewer splits if the launch would be more than a third larger than what
    fits on the GPU at once with four pages in flight per CTA (512 to 576 CTAs of four warps
    still beat half as many splits, 768 do not), and only counts that deal the pages out
    evenly (three splits of 16 pages measured 10 % worse than two or four).  More, while the
    launch is still smaller than the GPU.  `most`: the largest count allowed (what merges
    inside a thread-block cluster, or 16)."""
    four_pages = 8 * page * (head_dim + 8) * 2
    room = max(1, min(8, (228 * 1024) // (four_pages + 1024))) * sms
    most = max(1, min(pages, most))
    s = max(1, min(most, -(-pages // 4)))
    while s > 1 and (s * base_ctas > room * 13 // 10 or pages % s):
        s -= 1
    while 2 * s <= most and 2 * s * base_ctas <= sms and pages % (2 * s) == 0:
        s *= 2
    return s


class KernelError(RuntimeError):
    pass


def dtype_code(t: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[t]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t}") from None


def _ptr(t: torch.Tensor | None) -> int:
    """The tensor's address (0 for None); the entry points declare their pointer arguments."""
    return 0 if t is None else t.data_ptr()


try:    # the current stream's handle without building a Stream object (a few hundred ns)
    _raw_stream = torch._C._cuda_getCurrentRawStream
except AttributeError:   # pragma: no cover
    _raw_stream = None


def _check(t: torch.Tensor, name: str, dtype=None, ndim=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name}: expected a CUDA tensor, got device {t.device}")
    if not t.is_contiguous():
        raise KernelError(f"{name}: expected a contiguous tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name}: expected {ndim} dimensions, got {t.dim()}")


class CudaBackend:
    """Calls into the compiled library."""

    name = "cuda"

    def __init__(self):
        from . import build
        from .signatures import declare
        self.lib = build.load()
        declare(self.lib)
        self._device_index = torch.cuda.current_device()
        self.launches = 0  # kernels launched through this backend (for measurement reports)
        self._scratch = {}
        self._argmax_scratch = {}
        self._prefill_scr = {}
        # NIMBUS_B200_NO_TCGEN05=1 keeps large bf16 products on the CUDA-core kernel (debugging)
        self.use_tcgen05 = os.environ.get("NIMBUS_B200_NO_TCGEN05", "") in ("", "0")
        # NIMBUS_B200_STREAM=0 keeps a decode step's products on the kernel that streams weights
        # through registers (comparison runs)
        self.use_stream = os.environ.get("NIMBUS_B200_STREAM", "1") != "0"
        # NIMBUS_B200_ROWS=0/1/2: products of up to 128 rows on the kernel that cuts K among the
        # CTAs of a cluster: never / where it is the faster one (a long K over few columns) /
        # wherever it applies
        self.use_rows = int(os.environ.get("NIMBUS_B200_ROWS", "1") or 1)
        # NIMBUS_B200_DECODE_CLUSTERS=0: the splits of the bfloat16 decode attention merge through
        # scratch memory and a counter instead of a thread-block cluster's shared memory
        self._cluster_limit = int(self.lib.nb_attention_decode_cluster_limit())
        self._sms = torch.cuda.get_device_properties(self._device_index).multi_processor_count
        self.set_decode_clusters(int(os.environ.get("NIMBUS_B200_DECODE_CLUSTERS", "1") or 1))
        # NIMBUS_B200_OVERLAP=0/1: let a kernel's set-up and first weight fetch overlap the tail
        # of the kernel before it (programmatic dependent launch; on by default)
        self.set_overlap(os.environ.get("NIMBUS_B200_OVERLAP", "1") != "0")
        # NIMBUS_B200_PAIRS=0/1/2: large products on pairs of CTAs: never / where the cost
        # model prefers them (products of three waves of tiles and more) / wherever possible
        self.set_pairs(int(os.environ.get("NIMBUS_B200_PAIRS", "1") or 1))

    def set_pairs(self, mode) -> None:
        """Large products on pairs of CTAs sharing 256-row tiles (`cta_group::2`): 0/False off,
        1/True where the cost model prefers them, 2 wherever a paired kernel exists."""
        self.pairs = int(mode)
        self.lib.nb_gemm_tcgen05_use_pairs(self.pairs)

    def set_decode_clusters(self, on) -> None:
        """Whether 2 to 8 splits of the bfloat16 decode attention merge inside a thread-block
        cluster (the default) or through scratch memory like any other number of them."""
        self.decode_clusters = 1 if on else 0
        self.lib.nb_attention_decode_cluster_merge(self.decode_clusters)

    def set_overlap(self, on: bool) -> None:
        self.lib.nb_set_overlap((1 if on else 0))
        self.overlap = bool(on)

    # -- plumbing ---------------------------------------------------------------------
    def _stream(self) -> int:
        if _raw_stream is not None:
            return _raw_stream(self._device_index)
        return torch.cuda.current_stream().cuda_stream

    def _call(self, fn_name: str, *args) -> None:
        rc = getattr(self.lib, fn_name)(*args)
        self.launches += 1
        if rc != 0:
            msg = self.lib.nb_last_error().decode("utf-8", "replace")
            raise KernelError(f"{fn_name} failed ({rc}): {msg}")

    # -- row-wise ---------------------------------------------------------------------
    def embed_pos(self, tokens, pos, wte, wpe, out):
        _check(tokens, "tokens", torch.int32, 1)
        _check(pos, "pos", torch.int32, 1)
        _check(wte, "wte", None, 2)
        _check(out, "out", torch.float32, 2)
        if wpe is not None:
            _check(wpe, "wpe", wte.dtype, 2)
        n, d = out.shape
        if tokens.numel() < n or pos.numel() < n or wte.shape[1] != d:
            raise KernelError("embed_pos: shapes do not agree")
        self._call("nb_embed_pos", _ptr(tokens), _ptr(pos), _ptr(wte), _ptr(wpe),
                   dtype_code(wte.dtype), _ptr(out), n, d, self._stream())

    def layernorm(self, x, gamma, beta, eps, out, rows=None):
        _check(x, "x", torch.float32, 2)
        _check(gamma, "gamma", torch.float32, 1)
        if beta is not None:
            _check(beta, "beta", torch.float32, 1)
        _check(out, "out", None, 2)
        if rows is not None:
            _check(rows, "rows", torch.int32, 1)
        n, d = out.shape
        if x.shape[1] != d or gamma.numel() != d or (rows is None and x.shape[0] < n):
            raise KernelError("layernorm: shapes do not agree")
        self._call("nb_layernorm", _ptr(x), _ptr(rows), _ptr(gamma), _ptr(beta), _ptr(out),
                   dtype_code(out.dtype), n, d, eps, self._stream())

    # -- matrix products --------------------------------------------------------------
    def linear(self, x, w, bias, out, act=ACT_NONE, residual=None, norm=None):
        """out = act(norm(x) @ w.T + bias) (+ residual).  x [M,K], w [N,K], out [M,N].
        ``norm``: ``(gamma, beta, eps, act_dtype)`` asks for LayerNorm of the fp32 rows ``x``
        first; it is fused into the product where the kernel can, else run on its own."""
        _check(x, "x", None, 2)
        _check(w, "w", None, 2)
        _check(out, "out", None, 2)
        M, K = x.shape
        N = w.shape[0]
        if w.shape[1] != K or out.shape[0] != M or out.shape[1] != N:
            raise KernelError(f"linear: shapes do not agree: x {tuple(x.shape)}, w {tuple(w.shape)}, "
                              f"out {tuple(out.shape)}")
        if bias is not None:
            _check(bias, "bias", torch.float32, 1)
            if bias.numel() != N:
                raise KernelError("linear: bias length does not match")
        if residual is not None:
            _check(residual, "residual", torch.float32, 2)
            if residual.shape != out.shape:
                raise KernelError("linear: residual shape does not match")
        tensor_core = (x.dtype == torch.bfloat16 or norm is not None and norm[3] == torch.bfloat16) \
            and w.dtype == torch.bfloat16 and K % 8 == 0 and self.use_tcgen05
        # few rows: the weight-streaming kernel; from 17 rows on the tensor-core kernel streams
        # weights faster (TMA ring), where it applies
        skinny = (M <= FUSED_NORM_MAX_ROWS or (M <= SKINNY_MAX_ROWS and not tensor_core)) \
            and (K * 32 <= 220 * 1024 if w.dtype == torch.float32 else K % 8 == 0)
        # a decode step's products (at most 16 rows, bf16 weights): weights into shared memory
        # before the kernel waits for its predecessor, so that they stream across kernel ends
        if self.use_stream and M <= STREAM_MAX_ROWS and w.dtype == torch.bfloat16 and K % 8 == 0 \
                and (norm is None or norm[3] == torch.bfloat16):
            fused = norm is not None and self.lib.nb_gemm_stream_supported(M, N, K, 1)
            if fused or self.lib.nb_gemm_stream_supported(M, N, K, 0):
                if norm is not None and not fused:
                    h = torch.empty((M, K), device=x.device, dtype=norm[3])
                    self.layernorm(x, norm[0], norm[1], norm[2], h)
                    x, norm = h, None
                gamma, beta, eps = (norm[0], norm[1], norm[2]) if norm is not None else (None, None, 0.0)
                self._call("nb_gemm_stream", _ptr(x), dtype_code(x.dtype), _ptr(gamma), _ptr(beta), eps,
                           _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), dtype_code(out.dtype), M, N,
                           K, act, self._stream())
                return
        if skinny:
            if norm is not None and (M > FUSED_NORM_MAX_ROWS or N > FUSED_NORM_MAX_COLS
                                     or w.dtype != torch.bfloat16
                                     or not self.lib.nb_gemm_skinny_norm_supported(M, N, K)):
                h = torch.empty((M, K), device=x.device, dtype=norm[3])
                self.layernorm(x, norm[0], norm[1], norm[2], h)
                x, norm = h, None
            gamma, beta, eps = (norm[0], norm[1], norm[2]) if norm is not None else (None, None, 0.0)
            self._call("nb_gemm_skinny", _ptr(x), dtype_code(x.dtype), _ptr(gamma),
                       _ptr(beta), eps, _ptr(w), dtype_code(w.dtype), _ptr(bias),
                       _ptr(residual), _ptr(out), dtype_code(out.dtype), M, N,
                       K, act, self._stream())
            return
        if norm is not None:
            h = torch.empty((M, K), device=x.device, dtype=norm[3])
            self.layernorm(x, norm[0], norm[1], norm[2], h)
            x = h
        # up to 128 rows with a long K over few columns (the MLP's second product of a decode
        # step of a larger batch or of a short prompt): weights as the 128-row operand, K cut
        # among the CTAs of a cluster
        if self.use_tcgen05 and self.use_rows and M <= ROWS_MAX_ROWS and x.dtype == torch.bfloat16 \
                and w.dtype == torch.bfloat16 and (
                    self.lib.nb_gemm_tc_rows_preferred(M, N, K) if self.use_rows == 1
                    else self.lib.nb_gemm_tc_rows_supported(M, N, K)):
            self._call("nb_gemm_tc_rows", _ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out),
                       dtype_code(out.dtype), M, N, K, act, self._stream())
            return
        if self.use_tcgen05 and self.lib.nb_gemm_tcgen05_supported(
                dtype_code(x.dtype), dtype_code(w.dtype), M, N, K):
            self._call("nb_gemm_tcgen05", _ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out),
                       dtype_code(out.dtype), M, N, K, act,
                       self._stream())
            return
        self._call("nb_gemm_simt", _ptr(x), dtype_code(x.dtype), _ptr(w),
                   dtype_code(w.dtype), _ptr(bias), _ptr(residual), _ptr(out),
                   dtype_code(out.dtype), M, N, K, act,
                   self._stream())

    # A kernel whose bounded wait on a barrier ran out says so in a word of pinned host memory
    # (one per kernel family); its results are not valid.
    _ERROR_WORDS = {0: "gemm_tcgen05", 1: "attention_prefill_tc", 2: "wait_probe", 3: "gemm_stream",
                    4: "gemm_tc_rows"}

    def raise_device_errors(self) -> None:
        """Raise if a kernel that has finished reported a timed-out wait.  Reads host memory
        only: call it where the host has already waited for the work it hands out (logits
        copied to the host, sampled tokens read back)."""
        mask = self.lib.nb_device_errors(1)
        if mask:
            names = [self._ERROR_WORDS.get(i, f"word {i}") for i in range(16) if mask >> i & 1]
            raise KernelError(f"{', '.join(names)}: a wait on a shared-memory barrier ran out of "
                              "time; results of the steps since the last check are not valid")

    def check_device_errors(self) -> None:
        """Wait for the device, then raise if a kernel reported a timed-out wait."""
        torch.cuda.synchronize(self._device_index)
        self.raise_device_errors()

    def set_wait_budget(self, cycles: int | None) -> None:
        """Clock cycles a wait on a barrier may take in the tensor-core kernels before the
        kernel gives up and reports it (``None``: the default, about two seconds)."""
        cycles = 4_000_000_000 if cycles is None else int(cycles)
        for fn in ("nb_gemm_tcgen05_set_wait_budget", "nb_attention_prefill_tc_set_wait_budget",
                   "nb_gemm_stream_set_wait_budget", "nb_gemm_tc_rows_set_wait_budget"):
            rc = getattr(self.lib, fn)(cycles)
            if rc != 0:
                raise KernelError(f"{fn} failed ({rc}): "
                                  + self.lib.nb_last_error().decode("utf-8", "replace"))

    def wait_probe(self) -> int:
        """Run the kernels' bounded wait on a barrier that nothing completes; returns 2 if it
        gave up after the budget (the error word is then raised), 1 if it came back complete."""
        status = torch.zeros(1, dtype=torch.int32, device=f"cuda:{self._device_index}")
        self._call("nb_wait_probe", _ptr(status), self._stream())
        return int(status.item())

    # -- cache and attention ----------------------------------------------------------
    def _decode_splits(self, base_ctas: int, pages: int, kv, dtype) -> int:
        """Into how many splits a decode launch cuts each sequence's pages (`base_ctas`: rows x
        key-value heads).  The 32-bit kernel aims at a fixed number of CTAs; the tensor-core
        kernel follows `decode_splits`."""
        if dtype != torch.bfloat16:
            return max(1, min(pages, DECODE_TARGET_CTAS // base_ctas))
        return decode_splits(base_ctas, pages, kv.page, kv.head_dim, self._sms,
                             self._cluster_limit if self.decode_clusters else 16)

    def _decode_scratch(self, device, n_rows, n_heads, n_kv_heads, head_dim, n_splits):
        """Scratch of the split decode attention: partial sums per (row, head, split) and one
        counter per (row, key/value head).  Kept and grown as needed; the counters start at
        zero and every launch leaves them at zero."""
        need_acc = n_rows * n_heads * n_splits * head_dim
        need_ml = n_rows * n_heads * n_splits * 2
        need_cnt = n_rows * n_kv_heads
        s = self._scratch.get(device)
        if s is None or s[0].numel() < need_acc or s[1].numel() < need_ml or s[2].numel() < need_cnt:
            s = (torch.empty(max(need_acc, 1 << 16), dtype=torch.float32, device=device),
                 torch.empty(max(need_ml, 1 << 12), dtype=torch.float32, device=device),
                 torch.zeros(max(need_cnt, 1 << 12), dtype=torch.int32, device=device))
            self._scratch[device] = s
        return s

    def scratch_refs(self):
        """The scratch tensors kernels currently use: whoever records launches in a CUDA graph
        keeps these alive with it (growing a scratch buffer replaces the tensor)."""
        return (dict(self._scratch), dict(self._argmax_scratch), dict(self._prefill_scr))

    def _prefill_scratch(self, device, n_tiles, max_splits, head_dim):
        """Scratch of the split prefill attention: one record per (tile, split) and one counter
        per tile; the counters start at zero and every launch leaves them at zero."""
        rec = self.lib.nb_attention_prefill_tc_record(head_dim)
        need = n_tiles * max_splits * rec
        s = self._prefill_scr.get(device)
        if s is None or s[0].numel() < need or s[1].numel() < n_tiles:
            s = (torch.empty(max(need, 1 << 20), dtype=torch.float32, device=device),
                 torch.zeros(max(n_tiles, 1 << 12), dtype=torch.int32, device=device))
            self._prefill_scr[device] = s
        return s

    def kv_append(self, src, k_col, v_col, row_slot, row_pos, kv, n_rows):
        _check(src, "src", kv.k.dtype, 2)
        self._call("nb_kv_append", _ptr(src), dtype_code(src.dtype), src.shape[1],
                   k_col, v_col, _ptr(row_slot), _ptr(row_pos), _ptr(kv.k),
                   _ptr(kv.v), _ptr(kv.block_table), kv.block_table.shape[1],
                   kv.page, kv.n_kv_heads, kv.head_dim, n_rows,
                   self._stream())

    def attention(self, q_src, q_col, layout, kv, n_heads, out, scale, window=0, append=None):
        """Causal attention of the packed rows of ``layout`` over the cache ``kv``.
        ``append=(k_col, v_col)``: the rows of ``q_src`` also hold this step's keys and values
        at those columns; they are written to the cache as well (inside the decode kernel and,
        for sequences that start at a page boundary, inside the tensor-core prefill kernel;
        else by a pass of their own before the attention kernel)."""
        _check(q_src, "q", kv.k.dtype, 2)
        _check(out, "out", None, 2)
        n_rows = layout.n_rows
        if out.shape[0] < n_rows or out.shape[1] != n_heads * kv.head_dim:
            raise KernelError("attention: output shape does not match")
        if layout.is_decode and self.lib.nb_attention_decode_supported(
                dtype_code(q_src.dtype), kv.head_dim, n_heads,
                kv.n_kv_heads, kv.page):
            pages = max(1, -(-layout.max_kv_len // kv.page))
            n_splits = self._decode_splits(n_rows * kv.n_kv_heads, pages, kv, q_src.dtype)
            acc, ml, counters = self._decode_scratch(q_src.device, n_rows, n_heads, kv.n_kv_heads,
                                                     kv.head_dim, n_splits)
            self._call("nb_attention_decode", _ptr(q_src), dtype_code(q_src.dtype),
                       q_src.shape[1], q_col, _ptr(layout.row_slot),
                       _ptr(layout.row_pos), _ptr(kv.k), _ptr(kv.v), _ptr(kv.block_table),
                       kv.block_table.shape[1], kv.page, n_heads,
                       kv.n_kv_heads, kv.head_dim, _ptr(out),
                       dtype_code(out.dtype), out.shape[1], scale,
                       window, n_rows, n_splits, _ptr(acc), _ptr(ml),
                       _ptr(counters), (1 if append else 0),
                       (append[0] if append else 0), (append[1] if append else 0),
                       self._stream())
            return
        if (not layout.is_decode) and self.use_tcgen05 and scale > 0 and self.lib.nb_attention_prefill_tc_supported(
                dtype_code(q_src.dtype), kv.head_dim, n_heads, kv.n_kv_heads, kv.page,
                q_src.shape[1], q_col, dtype_code(out.dtype), out.shape[1]):
            # 5th-generation tensor cores, scores in tensor memory.  When every sequence's cached
            # length is a whole number of pages (prompts from their first token, chunks cut at
            # page ends) the kernel reads the step's keys and values from the step's rows and
            # writes them to the cache itself; else they are appended first.
            fused = bool(append) and append[0] % 8 == 0 and append[1] % 8 == 0 and \
                all(p % kv.page == 0 for p in layout.seq_pos0_host)
            if append and not fused:
                self.kv_append(q_src, append[0], append[1], layout.row_slot, layout.row_pos, kv, n_rows)
            if layout.n_rows > layout.n_tokens:
                out[layout.n_tokens:layout.n_rows].zero_()      # padding rows
            # A CTA takes a 128-row tile of one head.  When there are too few of them to fill
            # the GPU, the pages a tile reads are cut into up to four runs of at least four
            # pages, one CTA each, and merged by the CTA that finishes last.
            tiles = -(-layout.max_q_len // 128)
            ctas = tiles * n_heads * layout.n_seqs
            pages = -(-layout.max_kv_len // kv.page)
            if window > 0:
                pages = min(pages, (window + 127) // kv.page + 2)
            max_splits = 1
            if 2 * ctas <= PREFILL_TARGET_CTAS and pages >= 8:
                max_splits = min(4, PREFILL_TARGET_CTAS // ctas, pages // 4)
            chunk = -(-pages // max_splits)
            part = counters = None
            if max_splits > 1:
                part, counters = self._prefill_scratch(q_src.device, ctas, max_splits, kv.head_dim)
            self._call("nb_attention_prefill_tc", _ptr(q_src), dtype_code(q_src.dtype),
                       q_src.shape[1], q_col, q_src.shape[0], _ptr(layout.cu_rows),
                       _ptr(layout.seq_slot), _ptr(layout.seq_pos0), _ptr(kv.k), _ptr(kv.v),
                       kv.k.shape[0], _ptr(kv.block_table), kv.block_table.shape[1], kv.page,
                       n_heads, kv.n_kv_heads, kv.head_dim, _ptr(out), dtype_code(out.dtype),
                       out.shape[1], scale, window, layout.n_seqs, layout.max_q_len,
                       max_splits, chunk, _ptr(part), _ptr(counters), 1 if fused else 0,
                       append[0] if fused else 0, append[1] if fused else 0, self._stream())
            return
        if append:
            self.kv_append(q_src, append[0], append[1], layout.row_slot, layout.row_pos, kv, n_rows)
        if (not layout.is_decode) and self.lib.nb_attention_prefill_supported(
                dtype_code(q_src.dtype), kv.head_dim, n_heads,
                kv.n_kv_heads, kv.page, q_src.shape[1], q_col):
            if layout.n_rows > layout.n_tokens:
                out[layout.n_tokens:layout.n_rows].zero_()      # padding rows
            self._call("nb_attention_prefill", _ptr(q_src), dtype_code(q_src.dtype),
                       q_src.shape[1], q_col, _ptr(layout.cu_rows),
                       _ptr(layout.seq_slot), _ptr(layout.seq_pos0), _ptr(kv.k), _ptr(kv.v),
                       _ptr(kv.block_table), kv.block_table.shape[1], kv.page,
                       n_heads, kv.n_kv_heads, kv.head_dim, _ptr(out),
                       dtype_code(out.dtype), out.shape[1], scale,
                       window, layout.n_seqs, layout.max_q_len, self._stream())
            return
        if (not layout.is_decode) and q_src.dtype == torch.float32 and \
                self.lib.nb_attention_prefill_f32_supported(kv.head_dim, n_heads, kv.n_kv_heads, kv.page):
            # the 32-bit path's prompts: tiles of 64 rows, fp32 multiply-adds
            if layout.n_rows > layout.n_tokens:
                out[layout.n_tokens:layout.n_rows].zero_()      # padding rows
            self._call("nb_attention_prefill_f32", _ptr(q_src), dtype_code(q_src.dtype), q_src.shape[1],
                       q_col, _ptr(layout.cu_rows), _ptr(layout.seq_slot), _ptr(layout.seq_pos0),
                       _ptr(kv.k), _ptr(kv.v), _ptr(kv.block_table), kv.block_table.shape[1], kv.page,
                       n_heads, kv.n_kv_heads, kv.head_dim, _ptr(out), dtype_code(out.dtype),
                       out.shape[1], scale, window, layout.n_seqs, layout.max_q_len, self._stream())
            return
        self._call("nb_attention_generic", _ptr(q_src), dtype_code(q_src.dtype),
                   q_src.shape[1], q_col, _ptr(layout.row_slot), _ptr(layout.row_pos),
                   _ptr(kv.k), _ptr(kv.v), _ptr(kv.block_table), kv.block_table.shape[1],
                   kv.page, n_heads, kv.n_kv_heads, kv.head_dim,
                   _ptr(out), dtype_code(out.dtype), out.shape[1], scale,
                   window, n_rows, self._stream())

    def advance_decode(self, tokens, next_tokens, row_pos, row_slot):
        """tokens <- next_tokens, row_pos += 1 for live rows (between two decode steps)."""
        for t, n in ((tokens, "tokens"), (next_tokens, "next"), (row_pos, "row_pos"),
                     (row_slot, "row_slot")):
            _check(t, n, torch.int32, 1)
        self._call("nb_advance_decode", _ptr(tokens), _ptr(next_tokens), _ptr(row_pos),
                   _ptr(row_slot), (tokens.numel()), self._stream())

    # -- sampling ---------------------------------------------------------------------
    def argmax(self, logits, out):
        _check(logits, "logits", torch.float32, 2)
        _check(out, "out", torch.int32, 1)
        n, v = logits.shape
        n_ctas = min(32, max(1, v // 2048))
        if n_ctas > 1 and n * n_ctas <= 4096:
            s = self._argmax_scratch.get(logits.device)
            if s is None or s[0].numel() < n:
                s = (torch.zeros(max(n, 256), dtype=torch.int64, device=logits.device),
                     torch.zeros(max(n, 256), dtype=torch.int32, device=logits.device))
                self._argmax_scratch[logits.device] = s
            self._call("nb_argmax_split", _ptr(logits), n, v, _ptr(out), _ptr(s[0]),
                       _ptr(s[1]), n_ctas, self._stream())
            return
        self._call("nb_argmax", _ptr(logits), n, v, _ptr(out), self._stream())

    def sample_temperature(self, logits, temperature, u, out):
        _check(logits, "logits", torch.float32, 2)
        _check(u, "u", torch.float64, 1)
        _check(out, "out", torch.int32, 1)
        n, v = logits.shape
        self._call("nb_sample_temperature", _ptr(logits), n, v,
                   temperature, _ptr(u), _ptr(out), self._stream())

    def sample_top_k(self, logits, k, temperature, u, out):
        """Top-k sampling (no top-p) on the device: ``out[r]`` is drawn with ``u[r]`` among the
        row's ``k`` largest logits (ties at the k-th included); -1 marks a row with a NaN."""
        _check(logits, "logits", torch.float32, 2)
        _check(u, "u", torch.float64, 1)
        _check(out, "out", torch.int32, 1)
        n, v = logits.shape
        self._call("nb_sample_top_k", _ptr(logits), n, v, int(k), float(temperature), _ptr(u),
                   _ptr(out), self._stream())

    def top_p_max_k(self) -> int:
        """The largest top-k that :meth:`sample_top_p` takes together with top-p."""
        return int(self.lib.nb_sample_top_p_max_k())

    def sample_top_p(self, logits, k, top_p, temperature, u, out):
        """Top-p sampling (with top-k ``k``, 0 = off) on the device.  ``out[r]`` is the token,
        -1 for a row with a NaN, -2 for a row whose cut lies beyond the thousand largest logits
        (a flat distribution): those the caller settles on the host."""
        _check(logits, "logits", torch.float32, 2)
        _check(u, "u", torch.float64, 1)
        _check(out, "out", torch.int32, 1)
        n, v = logits.shape
        self._call("nb_sample_top_p", _ptr(logits), n, v, int(k), float(top_p), float(temperature),
                   _ptr(u), _ptr(out), self._stream())

    def top_candidates(self, logits, n_keep, temp):
        """The ``n_keep`` largest logits of every row with their indices (plus ties at the
        threshold, up to ``n_keep + 32``), the row maximum and the f64 sum of
        ``exp((x - max) / temp)`` over the row.  Returns ``(values [n, cap] f32, indices
        [n, cap] i32, counts [n] i32, stats [n, 2] f64)`` on the device; a count of -1 marks a
        row with a NaN, a count above ``cap`` ties that did not fit."""
        _check(logits, "logits", torch.float32, 2)
        n, v = logits.shape
        cap = n_keep + 32
        dev = logits.device
        vals = torch.empty((n, cap), dtype=torch.float32, device=dev)
        idx = torch.empty((n, cap), dtype=torch.int32, device=dev)
        counts = torch.empty(n, dtype=torch.int32, device=dev)
        stats = torch.empty((n, 2), dtype=torch.float64, device=dev)
        self._call("nb_top_candidates", _ptr(logits), n, v, n_keep, cap, float(temp), _ptr(vals),
                   _ptr(idx), _ptr(counts), _ptr(stats), self._stream())
        return vals, idx, counts, stats

    def history_append(self, history, history_len, tokens, row_slot):
        """history[r, history_len[r]] <- tokens[r], history_len[r] += 1 for live rows (a decode
        session's record of what each sequence has generated)."""
        _check(history, "history", torch.int32, 2)
        for t, n in ((history_len, "history_len"), (tokens, "tokens"), (row_slot, "row_slot")):
            _check(t, n, torch.int32, 1)
        self._call("nb_history_append", _ptr(history), history.shape[1], _ptr(history_len),
                   _ptr(tokens), _ptr(row_slot), tokens.numel(), self._stream())

    def repetition_penalty(self, logits, history, history_len, penalty):
        _check(logits, "logits", torch.float32, 2)
        _check(history, "history", torch.int32, 2)
        _check(history_len, "history_len", torch.int32, 1)
        n, v = logits.shape
        self._call("nb_repetition_penalty", _ptr(logits), n, v, _ptr(history),
                   history.shape[1], _ptr(history_len), penalty, self._stream())


_backend = None


def backend():
    """The installed backend; the CUDA library is loaded (and built) on first use."""
    global _backend
    if _backend is None:
        if not torch.cuda.is_available():
            raise KernelError(
                "no CUDA device: this library runs its models only through its sm_100a kernels "
                "and has no CPU path")
        _backend = CudaBackend()
    return _backend


def set_backend(b) -> None:
    """Install another backend object (tests of host logic) or ``None`` to reset."""
    global _backend
    _backend = b
