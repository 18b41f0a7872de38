"""A stand-in for the kernels, in plain torch on the CPU, for tests of the host side only.

The product has no CPU path: `Engine` takes its kernels from the CUDA extension and fails without
it.  This double has the same methods so that the tests that need no GPU can run the step
function, the cache and the generation loop against the plain implementation.  It is written for
clarity, reads the same packed step description and the same paged cache, and is not shipped.
"""
from __future__ import annotations

import math

import torch

PAGE = 64


class CpuOps:
    name = "cpu-double"

    def embed(self, tokens, positions, table, pos_table):
        x = table[tokens.long()].float()
        if pos_table is not None:
            x = x + pos_table[positions.long()].float()
        return x

    def layernorm(self, x, w, b, eps, out_dtype):
        x = x.float()
        mean = x.mean(-1, keepdim=True)
        var = ((x - mean) ** 2).mean(-1, keepdim=True)
        return ((x - mean) * torch.rsqrt(var + eps) * w + b).to(out_dtype)

    def linear(self, a, w, bias, act=None, residual=None, out_dtype=None):
        y = a.float() @ w.float().t()
        if bias is not None:
            y = y + bias
        if act == "gelu_tanh":
            y = 0.5 * y * (1 + torch.tanh(math.sqrt(2 / math.pi) * (y + 0.044715 * y ** 3)))
        elif act == "gelu_erf":
            y = 0.5 * y * (1 + torch.erf(y / math.sqrt(2)))
        elif act is not None:
            raise ValueError(act)
        if residual is not None:
            return residual + y
        return y.to(out_dtype)

    def clear_tails(self, group, tails):
        for page, row in tails.tolist():
            if page >= 0:
                for t in list(group.k) + list(group.v):
                    t[page, :, row:, :] = 0

    def kv_store(self, qkv, cache, plan, n_heads, kv_heads, head_dim):
        g = cache.group_index
        q_w = n_heads * head_dim
        kv_w = kv_heads * head_dim
        for t in range(plan.T):
            s = int(plan.token_seq[t])
            if int(plan.seq_slot[s]) < 0:
                continue
            p = int(plan.positions[t])
            page = int(plan.pages[g][s, p // PAGE])
            assert page >= 0, "a position is written whose page is not held"
            cache.k[page, :, p % PAGE, :] = qkv[t, q_w:q_w + kv_w].view(kv_heads, head_dim).to(cache.k.dtype)
            cache.v[page, :, p % PAGE, :] = qkv[t, q_w + kv_w:].view(kv_heads, head_dim).to(cache.v.dtype)

    def attention(self, qkv, cache, plan, n_heads, kv_heads, head_dim, scale, window, out_dtype, store=False):
        if store:
            self.kv_store(qkv, cache, plan, n_heads, kv_heads, head_dim)
        g = cache.group_index
        out = torch.zeros(plan.T, n_heads * head_dim)
        rep = n_heads // kv_heads
        for t in range(plan.T):
            s = int(plan.token_seq[t])
            if int(plan.seq_slot[s]) < 0:
                continue
            p = int(plan.positions[t])
            lo = max(0, p - window + 1) if window > 0 else 0
            pos = torch.arange(lo, p + 1)
            pages = plan.pages[g][s, pos // PAGE].long()
            assert (pages >= 0).all(), "a position is read whose page is not held"
            k = cache.k[pages, :, pos % PAGE, :].float()      # [keys, kv_heads, hd]
            v = cache.v[pages, :, pos % PAGE, :].float()
            q = qkv[t, :n_heads * head_dim].float().view(n_heads, head_dim)
            for h in range(n_heads):
                sc = (k[:, h // rep, :] @ q[h]) * scale
                pr = torch.softmax(sc, 0)
                out[t, h * head_dim:(h + 1) * head_dim] = pr @ v[:, h // rep, :]
        return out.to(out_dtype)

    def scale_cap(self, x, scale=1.0, cap=None):
        x.mul_(scale)
        if cap is not None:
            x.copy_(cap * torch.tanh(x / cap))
        return x

    def take_tokens(self, tokens, token_src, ids, vocab_size):
        take = token_src >= 0
        tokens[take] = ids[token_src[take].long()].to(tokens.dtype)

    def gather_rows(self, x, rows, n_rows):
        return x[rows[:n_rows].long()]

    def sample(self, logits, temperature, top_k, top_p, seed, streams, counters):
        import plain_gpt2
        out = [plain_gpt2.sample(logits[r].double().numpy(), temperature, top_k, top_p,
                                 plain_gpt2.uniform01(seed, int(streams[r]), int(counters[r])))
               for r in range(logits.shape[0])]
        return torch.tensor(out, dtype=torch.int32)
