"""A stand-in for the kernel library with the same methods, computed with torch on the CPU.

It exists so that the host-side logic (step tables, cache manager, scheduler, engine) can be exercised by the
tests that run without a GPU. It is test code only: the package has no CPU path and never imports this.
"""
from __future__ import annotations

import math

import torch

from tests.plain import qwen3_plain as plain


class FakeKernels:
    launches = 0
    library_launches = 0

    def embedding(self, table, ids):
        return table[ids.long()].clone()

    def rms_norm(self, x, w, eps, rows=None):
        if rows is not None:
            x = x[rows.long()]
        xf = x.float()
        y = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps) * w.float()
        return y.to(x.dtype)

    def add_rms_norm(self, x, residual, w, eps, rows=None):
        s = (x.float() + residual.float()).to(x.dtype)
        if rows is None:
            residual.copy_(s)
        return self.rms_norm(s, w, eps, rows)

    def silu_mul(self, x, block=0):
        i = x.shape[1] // 2
        if block:
            x = x.reshape(x.shape[0], i // block, 2, block).permute(0, 2, 1, 3).reshape(x.shape[0], 2 * i)
        g, u = x[:, :i].float(), x[:, i:].float()
        return (g / (1 + torch.exp(-g)) * u).to(x.dtype)

    def qk_norm_rope_cache(self, qkv, q_heads, kv_heads, head_dim, *, q_w, k_w, eps, inv_freq, rotary_dim, positions,
                           k_pool=None, v_pool=None, slot_mapping=None, page_size=0, write_kv=True, cos_sin=None):
        T = qkv.shape[0]
        d = head_dim
        q = qkv[:, : q_heads * d].reshape(T, q_heads, d).float()

        def norm(x, w):
            return x if w is None else x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w.float()

        def rope(x):
            if not rotary_dim:
                return x
            half = rotary_dim // 2
            if cos_sin is not None:     # the step's own table of cosines and sines [T, half, 2]
                c, s = cos_sin[:, None, :, 0].float(), cos_sin[:, None, :, 1].float()
            else:
                ang = positions.double()[:, None] * inv_freq[None, :]
                c, s = torch.cos(ang)[:, None, :].float(), torch.sin(ang)[:, None, :].float()
            x1, x2 = x[..., :half], x[..., half:rotary_dim]
            out = x.clone()
            out[..., :half] = x1 * c - x2 * s
            out[..., half:rotary_dim] = x2 * c + x1 * s
            return out

        q = rope(norm(q, q_w)).to(qkv.dtype)
        if write_kv:
            k = qkv[:, q_heads * d : (q_heads + kv_heads) * d].reshape(T, kv_heads, d).float()
            v = qkv[:, (q_heads + kv_heads) * d :].reshape(T, kv_heads, d)
            k = rope(norm(k, k_w)).to(qkv.dtype)
            for t in range(T):
                slot = int(slot_mapping[t])
                if slot < 0:
                    continue
                page, off = divmod(slot, page_size)
                k_pool[page, :, off, :] = k[t]
                v_pool[page, :, off, :] = v[t]
        return q.contiguous()

    def paged_attention_generic(self, q, k_pool, v_pool, positions, token_row, kv_indptr, kv_indices, scale, window):
        T, nq, d = q.shape
        nkv, page = k_pool.shape[1], k_pool.shape[2]
        group = nq // nkv
        out = torch.zeros(T, nq * d, dtype=q.dtype)
        for t in range(T):
            pos = int(positions[t])
            b = int(token_row[t])
            pages = kv_indices[int(kv_indptr[b]) : int(kv_indptr[b + 1])]
            lo = max(0, pos - window + 1) if window else 0
            js = list(range(lo, pos + 1))
            kk = torch.stack([k_pool[int(pages[j // page]), :, j % page, :] for j in js]).float()  # [n, nkv, d]
            vv = torch.stack([v_pool[int(pages[j // page]), :, j % page, :] for j in js]).float()
            for h in range(nq):
                s = (kk[:, h // group, :] @ q[t, h].float()) * scale
                p = torch.softmax(s, 0)
                out[t, h * d : (h + 1) * d] = (p @ vv[:, h // group, :]).to(q.dtype)
        return out

    def gemm_stream_supported(self, *a):
        return False

    def gemm_stream_swiglu_supported(self, *a):
        return False

    def gemm_simt(self, a, w, out_dtype=None):
        return (a.float() @ w.float().t()).to(out_dtype or a.dtype)

    def argmax(self, logits):
        return torch.tensor([plain.sample_row(r.tolist(), 0.0) for r in logits], dtype=torch.int32)

    def sample_penalise(self, logits, counts, prompt_bits, row_slot, repetition, presence, frequency, mask_bits=None):
        out = logits.clone()
        V = logits.shape[1]
        for r in range(logits.shape[0]):
            slot = int(row_slot[r])
            if slot < 0:
                continue
            c = {v: int(n) for v, n in enumerate(counts[slot].tolist()) if n}
            words = prompt_bits[slot].tolist()
            prompt = [v for v in range(V) if (words[v >> 5] >> (v & 31)) & 1]
            out[r] = torch.tensor(plain.penalise_row(logits[r].tolist(), c, prompt, float(repetition[r]), float(frequency[r]), float(presence[r])))
            if mask_bits is not None:
                allowed = mask_bits[slot].tolist()
                for v in range(V):
                    if not (allowed[v >> 5] >> (v & 31)) & 1:
                        out[r, v] = float("-inf")
        return out

    def sample_count_tokens(self, counts, row_slot, ids):
        for r in range(ids.numel()):
            if int(row_slot[r]) >= 0 and 0 <= int(ids[r]) < counts.shape[1]:
                counts[int(row_slot[r]), int(ids[r])] += 1

    def sample_prompt_bits(self, bits_of_slot, ids):
        for v in ids.tolist():
            if 0 <= v < bits_of_slot.numel() * 32:
                word = int(bits_of_slot[v >> 5]) & 0xffffffff
                word |= 1 << (v & 31)
                bits_of_slot[v >> 5] = word - (1 << 32) if word >= (1 << 31) else word

    def sample_logprobs(self, logits, ids, top=0):
        lp = torch.tensor([plain.logprob_at(logits[r].tolist(), int(ids[r])) for r in range(logits.shape[0])], dtype=torch.float32)
        pairs = [plain.top_logprobs(logits[r].tolist(), top) for r in range(logits.shape[0])]
        R = logits.shape[0]
        return (lp, torch.tensor([p[0] for p in pairs], dtype=torch.int32).reshape(R, top),
                torch.tensor([p[1] for p in pairs], dtype=torch.float32).reshape(R, top))

    def sample(self, logits, temperature, top_k, top_p, min_p, seeds, offsets, workspace=None):
        out = []
        for r in range(logits.shape[0]):
            out.append(plain.sample_row(logits[r].tolist(), float(temperature[r]), int(top_k[r]), float(top_p[r]), float(min_p[r]),
                                        int(seeds[r]) & ((1 << 64) - 1), int(offsets[r])))
        return torch.tensor(out, dtype=torch.int32)
