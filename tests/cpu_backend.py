"""A stand-in for the kernel library, written with torch CPU ops, for tests of the engine's
HOST logic (batch packing, paging, slots, generation decisions) on a machine without a GPU.
It is a test double only: the package never installs it, and the GPU tests never use it.
Each method has the signature of the same-named method of ``csrc.ops.CudaBackend``.
"""
from __future__ import annotations

import math

import torch


class CpuBackend:
    name = "cpu-test-double"

    def __init__(self):
        self.launches = 0

    def embed_pos(self, tokens, pos, wte, wpe, out):
        n = out.shape[0]
        tok = tokens[:n].long()
        valid = tok >= 0
        x = wte[tok.clamp(min=0)].float()
        if wpe is not None:
            x = x + wpe[pos[:n].long()].float()
        out.copy_(torch.where(valid[:, None], x, torch.zeros_like(x)))

    def layernorm(self, x, gamma, beta, eps, out, rows=None):
        n = out.shape[0]
        src = x[:n] if rows is None else x[rows[:n].long().clamp(min=0)]
        mean = src.mean(-1, keepdim=True)
        var = ((src - mean) ** 2).mean(-1, keepdim=True)
        y = (src - mean) / torch.sqrt(var + eps) * gamma
        if beta is not None:
            y = y + beta
        if rows is not None:
            y = torch.where((rows[:n] >= 0)[:, None], y, torch.zeros_like(y))
        out.copy_(y.to(out.dtype))

    def linear(self, x, w, bias, out, act=0, residual=None, norm=None):
        if norm is not None:
            h = torch.empty(x.shape, dtype=norm[3])
            self.layernorm(x, norm[0], norm[1], norm[2], h)
            x = h
        y = x.float() @ w.float().t()
        if bias is not None:
            y = y + bias
        if act == 1:
            y = 0.5 * y * (1 + torch.tanh(0.7978845608028654 * (y + 0.044715 * y ** 3)))
        elif act == 2:
            y = 0.5 * y * (1 + torch.erf(y / math.sqrt(2.0)))
        if residual is not None:
            y = y + residual
        out.copy_(y.to(out.dtype))

    def kv_append(self, src, k_col, v_col, row_slot, row_pos, kv, n_rows):
        w = kv.n_kv_heads * kv.head_dim
        for r in range(n_rows):
            slot = int(row_slot[r])
            if slot < 0:
                continue
            pos = int(row_pos[r])
            page = int(kv.block_table[slot, pos // kv.page])
            kv.k[page, :, pos % kv.page, :] = src[r, k_col:k_col + w].view(kv.n_kv_heads, kv.head_dim)
            kv.v[page, :, pos % kv.page, :] = src[r, v_col:v_col + w].view(kv.n_kv_heads, kv.head_dim)

    def attention(self, q_src, q_col, layout, kv, n_heads, out, scale, window=0, append=None):
        if append:
            self.kv_append(q_src, append[0], append[1], layout.row_slot, layout.row_pos, kv,
                           layout.n_rows)
        hd, group = kv.head_dim, n_heads // kv.n_kv_heads
        for r in range(layout.n_rows):
            slot = int(layout.row_slot[r])
            if slot < 0:
                out[r].zero_()
                continue
            pos = int(layout.row_pos[r])
            lo = max(0, pos + 1 - window) if window > 0 else 0
            idx = torch.arange(lo, pos + 1)
            pages = kv.block_table[slot, (idx // kv.page).long()].long()
            within = (idx % kv.page).long()
            keys = kv.k[pages, :, within, :].float()      # [n, Hk, hd]
            vals = kv.v[pages, :, within, :].float()
            q = q_src[r, q_col:q_col + n_heads * hd].float().view(n_heads, hd)
            for h in range(n_heads):
                s = (keys[:, h // group] @ q[h]) * scale
                p = torch.softmax(s, dim=0)
                out[r, h * hd:(h + 1) * hd] = (p @ vals[:, h // group]).to(out.dtype)

    def argmax(self, logits, out):
        out.copy_(torch.argmax(logits, dim=-1).to(torch.int32))

    def sample_temperature(self, logits, temperature, u, out):
        w = logits.double() / max(temperature, 1e-6)
        e = torch.exp(w - w.max(-1, keepdim=True).values)
        c = torch.cumsum(e, -1)
        r = u[:, None] * c[:, -1:]
        idx = (c < r).sum(-1).clamp(max=logits.shape[1] - 1)
        out.copy_(idx.to(torch.int32))

    # The sampling kernels' stand-ins draw with the host's sampler and the number they are given.
    # `hand_back`: mark every row as the top-p kernel marks a row it cannot settle (-2).
    hand_back = False

    def _draw(self, logits, u, out, **kw):
        from nimbus_infer_rs_b200.sampling import SamplingParams
        from nimbus_infer_rs_b200.sampling import host as H
        from nimbus_infer_rs_b200.sampling.device import _Drawn
        p = SamplingParams(**kw)
        for r in range(logits.shape[0]):
            out[r] = int(H.sample(logits[r].numpy(), p, [], _Drawn(float(u[r]))))

    def sample_top_k(self, logits, k, temperature, u, out):
        self._draw(logits, u, out, temperature=temperature, top_k=k)

    def top_p_max_k(self):
        return 1024

    def sample_top_p(self, logits, k, top_p, temperature, u, out):
        if self.hand_back:
            out.fill_(-2)
        else:
            self._draw(logits, u, out, temperature=temperature, top_k=k, top_p=top_p)

    def history_append(self, history, history_len, tokens, row_slot):
        for r in range(tokens.numel()):
            if int(row_slot[r]) >= 0 and int(history_len[r]) < history.shape[1]:
                history[r, int(history_len[r])] = tokens[r]
                history_len[r] += 1

    def repetition_penalty(self, logits, history, history_len, penalty):
        for r in range(logits.shape[0]):
            for tok in set(history[r, :int(history_len[r])].tolist()):
                if 0 <= tok < logits.shape[1]:
                    v = logits[r, tok]
                    logits[r, tok] = v / penalty if v > 0 else v * penalty

    def raise_device_errors(self):
        pass

    def check_device_errors(self):
        pass

    def advance_decode(self, tokens, next_tokens, row_pos, row_slot):
        live = row_slot >= 0
        tokens.copy_(torch.where(live, next_tokens, torch.full_like(tokens, -1)))
        row_pos.add_(live.to(row_pos.dtype))
