"""Plain PyTorch statement of every kernel, with the kernels' own calling convention.

Each method computes in float32 what the CUDA kernel of the same name computes, on
the same paged cache layout, one token at a time.  The GPU tests compare each
kernel with its method here on sizes other than the engine's; the CPU tests run
the engine's host logic (step function, cache manager, scheduler) through these
methods instead of CUDA.  This class lives under tests/: the engine itself has no
CPU path.
"""
from __future__ import annotations

import torch

F32 = torch.float32


class RefOps:
    name = "reference"

    def check_status(self):
        pass

    # ---- weights -------------------------------------------------------------------------
    def pack_linear(self, w):
        return w.contiguous()

    def pack_gate_up(self, gate, up):
        return torch.cat([gate, up], dim=0).contiguous()

    # ---- elementwise / rowwise -----------------------------------------------------------
    def embed(self, table, token_ids, out):
        out.copy_(table[token_ids.long()].to(F32))

    def rmsnorm(self, x, weight, eps, out, rows=None):
        src = x if rows is None else x[rows.long()]
        src = src.to(F32)
        inv = torch.rsqrt((src * src).mean(dim=-1, keepdim=True) + eps)
        out.copy_((src * inv * weight.to(F32)).to(out.dtype))

    def flush(self):
        pass

    def linear(self, a, w, out, accumulate=False, may_defer=False):
        prod = a.to(F32) @ w.to(F32).T
        if accumulate:
            out.add_(prod)
        else:
            out.copy_(prod)

    def gate_up_swiglu(self, h, w_gate_up, out):
        inter = out.shape[1]
        gu = h.to(F32) @ w_gate_up.to(F32).T
        gate, up = gu[:, :inter], gu[:, inter:]
        out.copy_((gate / (1.0 + torch.exp(-gate)) * up).to(out.dtype))

    def swiglu_ffn(self, h, w_gate_up, w_down, residual, may_defer=False):
        y = torch.empty((h.shape[0], w_down.shape[1]), dtype=h.dtype, device=h.device)
        self.gate_up_swiglu(h, w_gate_up, y)
        self.linear(y, w_down, residual, accumulate=True)

    # ---- attention -----------------------------------------------------------------------
    def qk_norm_rope_store(self, qkv, q_weight, k_weight, eps, rotation, step, cache, q_out,
                           num_heads, num_kv_heads, head_dim):
        """``rotation``: kind "neox" (half-split pairs over the first ``rotary_dim`` elements of a
        head, the rest left alone) or "none"."""
        assert rotation.kind in ("neox", "none"), rotation.kind
        t = qkv.shape[0]
        nq, nk = num_heads * head_dim, num_kv_heads * head_dim
        rot = int(rotation.rotary_dim)
        half = rot // 2
        q = qkv[:, :nq].reshape(t, num_heads, head_dim).to(F32)
        k = qkv[:, nq:nq + nk].reshape(t, num_kv_heads, head_dim).to(F32)
        v = qkv[:, nq + nk:].reshape(t, num_kv_heads, head_dim).to(F32)

        def norm(x, w):
            return x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w.to(F32)

        def rot_heads(x):
            if rot == 0:
                return x
            ang = step.positions.to(F32)[:, None] * rotation.inv_freq.to(F32)[None, :]
            c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
            x0, x1 = x[..., :half], x[..., half:rot]
            return torch.cat([x0 * c - x1 * s, x0 * s + x1 * c, x[..., rot:]], dim=-1)

        q = rot_heads(norm(q, q_weight))
        k = rot_heads(norm(k, k_weight))
        q_out.copy_(q.reshape(t, nq).to(q_out.dtype))
        if cache.writes:
            ps = cache.page_size
            pos = step.positions.long()
            page = cache.block_table[step.req_of_tok.long(), pos // ps].long()
            cache.pages[page, 0, :, pos % ps, :] = k.to(cache.pages.dtype)
            cache.pages[page, 1, :, pos % ps, :] = v.to(cache.pages.dtype)

    def qkv_rope_store(self, h, w_qkv, q_weight, k_weight, eps, rotation, step, cache, q_out,
                       num_heads, num_kv_heads, head_dim):
        qkv = torch.empty((q_out.shape[0], w_qkv.shape[0]), dtype=F32, device=q_out.device)
        self.linear(h, w_qkv, qkv)
        self.qk_norm_rope_store(qkv, q_weight, k_weight, eps, rotation, step, cache, q_out,
                                num_heads, num_kv_heads, head_dim)

    def qkv_attention(self, h, w_qkv, q_weight, k_weight, eps, rotation, step, cache, out,
                      num_heads, num_kv_heads, head_dim, window, scale):
        q = torch.empty((h.shape[0], num_heads * head_dim), dtype=h.dtype, device=h.device)
        self.qkv_rope_store(h, w_qkv, q_weight, k_weight, eps, rotation, step, cache, q,
                            num_heads, num_kv_heads, head_dim)
        self.paged_attention(q, step, cache, out, num_heads, num_kv_heads, head_dim, window, scale)

    def paged_attention(self, q, step, cache, out, num_heads, num_kv_heads, head_dim, window,
                        scale):
        t = q.shape[0]
        group = num_heads // num_kv_heads
        ps = cache.page_size
        qf = q.to(F32).reshape(t, num_heads, head_dim)
        res = torch.empty_like(qf)
        positions = step.positions.tolist()
        reqs = step.req_of_tok.tolist()
        for i in range(t):
            pos, r = positions[i], reqs[i]
            lo = 0 if window is None else max(0, pos - window + 1)
            p = torch.arange(lo, pos + 1, device=q.device)
            page = cache.block_table[r, p // ps].long()
            k = cache.pages[page, 0, :, p % ps, :].to(F32)        # [P, kv, hd]
            v = cache.pages[page, 1, :, p % ps, :].to(F32)
            k = k.repeat_interleave(group, dim=1)                # [P, heads, hd]
            v = v.repeat_interleave(group, dim=1)
            scores = torch.einsum("hd,phd->hp", qf[i], k) * scale
            prob = torch.softmax(scores, dim=-1)
            res[i] = torch.einsum("hp,phd->hd", prob, v)
        out.copy_(res.reshape(t, num_heads * head_dim).to(out.dtype))

    # ---- sampling ------------------------------------------------------------------------
    def argmax(self, logits, out):
        # first maximum wins ties
        mx = logits.max(dim=-1, keepdim=True).values
        idx = torch.arange(logits.shape[1], device=logits.device).expand_as(logits)
        big = torch.full_like(idx, logits.shape[1])
        out.copy_(torch.where(logits == mx, idx, big).min(dim=-1).values.to(out.dtype))

    def sample(self, logits, temperature, top_k, top_p, uniform, out):
        """Sort-based statement of the sampling kernel's rule (see csrc/sampling.cu)."""
        for r in range(logits.shape[0]):
            x = logits[r].double()
            t = float(temperature[r])
            if not t > 0.0:
                out[r] = int((x == x.max()).nonzero()[0])
                continue
            keep = torch.ones_like(x, dtype=torch.bool)
            k = int(top_k[r])
            if 0 < k < x.numel():
                keep &= x >= torch.sort(x, descending=True).values[k - 1]
            e = torch.where(keep, torch.exp((x - x.max()) / t), torch.zeros_like(x))
            p = float(top_p[r])
            if p < 1.0:
                vals, order = torch.sort(e, descending=True, stable=True)
                cum = torch.cumsum(vals, 0)
                cut = int((cum >= p * e.sum()).nonzero()[0])
                keep &= x >= x[order[cut]]
                e = torch.where(keep, e, torch.zeros_like(e))
            run = torch.cumsum(e, 0)
            hit = (run > float(uniform[r]) * e.sum()).nonzero()
            out[r] = int(hit[0]) if hit.numel() else int(keep.nonzero()[-1])
