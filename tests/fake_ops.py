"""A torch stand-in for the kernel pack, for tests of HOST-SIDE logic on the CPU.

The product has no CPU path.  This file lets the tests that run without a
GPU drive the real config, loader, parts, cache manager, batch builder,
step function and scheduler, so that faults in block tables, slot mappings
and request bookkeeping show up before a GPU is involved.  It mirrors the
method names of ``pih_b200.kernels.ops.CudaOps`` and nothing else of it.
"""
import torch


class FakeOps:
    launches = 0

    def __init__(self):
        self.error_word = torch.zeros(1, dtype=torch.int32)      # as the kernels' error word: first fault stays

    def _report(self, code):
        if int(self.error_word) == 0:
            self.error_word[0] = code

    def clear_errors(self):
        self.error_word.zero_()

    def check_errors(self):
        code = int(self.error_word)
        if code:
            self.clear_errors()
            raise RuntimeError(f"a kernel reported error code {code}")

    def embedding(self, table, ids):
        return table[ids.long()].clone()

    def rmsnorm(self, x, weight, eps, delta=None, rows=None):
        if rows is not None:
            v = x[rows.long()].float()
            if delta is not None:
                v = (v + delta[rows.long()].float()).to(x.dtype).float()
        else:
            v = x.float()
            if delta is not None:
                v = (v + delta.float()).to(x.dtype).float()
                x.copy_(v.to(x.dtype))
        scale = torch.rsqrt((v * v).sum(-1, keepdim=True) / v.shape[-1] + eps)
        return ((v * scale) * weight.float()).to(x.dtype)

    def linear(self, x, w, out_dtype=None):
        return (x.float() @ w.float().T).to(out_dtype or x.dtype)

    def qk_norm_rope_kv_write(self, qkv, *, heads, kv_heads, head_dim, q_norm, k_norm, eps, rope_table,
                              rotary_dim, positions, slot_mapping, kv_cache, write_kv):
        T = qkv.shape[0]
        D = head_dim
        page_size = kv_cache.shape[3]

        def norm_rope(x, w):                      # x [T, n, D]
            v = x.float()
            if w is not None:
                scale = torch.rsqrt((v * v).sum(-1, keepdim=True) / D + eps)
                v = ((v * scale) * w.float()).to(x.dtype).float()
            if rope_table is not None:
                cs = rope_table[positions.long()]        # [T, rot/2, 2]
                c, s = cs[..., 0][:, None, :], cs[..., 1][:, None, :]
                half = rotary_dim // 2
                a, b = v[..., :half], v[..., half:rotary_dim]
                v = torch.cat([a * c - b * s, b * c + a * s, v[..., rotary_dim:]], dim=-1)
            return v.to(x.dtype)

        q = qkv[:, :heads * D].reshape(T, heads, D)
        qkv[:, :heads * D] = norm_rope(q, q_norm).reshape(T, heads * D)
        if not write_kv:
            return
        k = qkv[:, heads * D:(heads + kv_heads) * D].reshape(T, kv_heads, D)
        v = qkv[:, (heads + kv_heads) * D:].reshape(T, kv_heads, D)
        k = norm_rope(k, k_norm)
        qkv[:, heads * D:(heads + kv_heads) * D] = k.reshape(T, kv_heads * D)
        sm = slot_mapping.long()
        assert (sm >= 0).all()
        page, off = sm // page_size, sm % page_size
        kv_cache[page, 0, :, off, :] = k
        kv_cache[page, 1, :, off, :] = v

    def paged_attention(self, qkv, *, heads, kv_heads, head_dim, kv_cache, block_table, step, scale, window):
        T, D = qkv.shape[0], head_dim
        page_size = kv_cache.shape[3]
        out = torch.zeros(T, heads, D, dtype=torch.float32)
        group = heads // kv_heads
        for t in range(T):
            r = int(step.request_of_row[t])
            p = int(step.positions[t])
            first = max(0, p - window + 1) if window else 0
            js = torch.arange(first, p + 1)
            pages = block_table[r, (js // page_size).long()].long()
            if not (pages >= 0).all():              # as the kernels: report "a row maps to no cache page", go on
                self._report(2)
                pages = pages.clamp(min=0)
            K = kv_cache[pages, 0, :, (js % page_size).long(), :].float()      # [n, kvh, D]
            V = kv_cache[pages, 1, :, (js % page_size).long(), :].float()
            q = qkv[t, :heads * D].reshape(heads, D).float()
            for h in range(heads):
                s = (K[:, h // group, :] @ q[h]) * scale
                out[t, h] = torch.softmax(s, dim=0) @ V[:, h // group, :]
        return out.reshape(T, heads * D).to(qkv.dtype)

    def silu_mul(self, gate_up, interleave=None):
        inter = gate_up.shape[1] // 2
        il = interleave or inter
        blocks = gate_up.reshape(gate_up.shape[0], inter // il, 2, il).float()
        g, u = blocks[:, :, 0, :].reshape(-1, inter), blocks[:, :, 1, :].reshape(-1, inter)
        return ((g / (1.0 + torch.exp(-g))) * u).to(gate_up.dtype)

    def norm_linear(self, h, delta, norm_weight, eps, w, swiglu_interleave=0):
        xn = self.rmsnorm(h, norm_weight, eps, delta=delta)
        out = self.linear(xn, w)
        if swiglu_interleave:
            out = self.silu_mul(out, swiglu_interleave)
        return h, out

    def argmax(self, logits):
        return torch.argmax(logits, dim=-1).to(torch.int32)

    def selected_logprob(self, logits, tokens, fparams=None, iparams=None):
        out = []
        for i in range(logits.shape[0]):
            t = float(fparams[i, 0]) if fparams is not None else 0.0
            scaled = logits[i].double() / (t if t > 0 else 1.0)
            keep = torch.ones(logits.shape[1], dtype=torch.bool)
            if iparams is not None:
                nsup = int(iparams[i, 5])
                keep[[int(v) for v in iparams[i, 6:6 + nsup].tolist()]] = False
            out.append(float(scaled[int(tokens[i])] - torch.logsumexp(scaled[keep], dim=0)))
        return torch.tensor(out, dtype=torch.float32)

    def top_logprobs(self, logits, count, fparams=None, iparams=None):
        from plain_impl import top_logprobs
        ids, lps = [], []
        for i in range(logits.shape[0]):
            t = float(fparams[i, 0]) if fparams is not None else 0.0
            nsup = int(iparams[i, 5]) if iparams is not None else 0
            sup = [int(v) for v in iparams[i, 6:6 + nsup].tolist()] if nsup else []
            top = top_logprobs(logits[i].tolist(), count, temperature=t, suppressed=sup)
            ids.append([a for a, _ in top])
            lps.append([b for _, b in top])
        return torch.tensor(ids, dtype=torch.int32), torch.tensor(lps, dtype=torch.float32)

    def sample(self, logits, fparams, iparams):
        from plain_impl import sample
        out = []
        for i in range(logits.shape[0]):
            ip = [int(v) & 0xFFFFFFFF for v in iparams[i].tolist()]
            nsup = ip[5]
            tok, _, _ = sample(logits[i].tolist(), temperature=float(fparams[i, 0]), top_p=float(fparams[i, 1]),
                               top_k=ip[0] or None, seed=ip[1] | (ip[2] << 32), ordinal=ip[3] | (ip[4] << 32),
                               suppressed=[int(v) for v in iparams[i, 6:6 + nsup].tolist()])
            out.append(tok)
        return torch.tensor(out, dtype=torch.int32)
