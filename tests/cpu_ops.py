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

    def embed(self, tokens, positions, table, pos_table, token_scale=1.0):
        x = table[tokens.long()].float() * token_scale
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
        elif act == "relu2":
            y = torch.relu(y) ** 2
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

    def kv_store(self, qkv, cache, plan, n_heads, kv_heads, head_dim, value_dim=None):
        g = cache.group_index
        q_w = n_heads * head_dim
        kv_w = kv_heads * head_dim
        vd = head_dim if value_dim is None else value_dim
        for t in range(plan.T):
            s = int(plan.token_seq[t])
            if int(plan.seq_slot[s]) < 0:
                continue
            p = int(plan.positions[t])
            page = int(plan.pages[g][s, p // PAGE])
            assert page >= 0, "a position is written whose page is not held"
            cache.k[page, :, p % PAGE, :] = qkv[t, q_w:q_w + kv_w].view(kv_heads, head_dim).to(cache.k.dtype)
            cache.v[page, :, p % PAGE, :] = qkv[t, q_w + kv_w:q_w + kv_w + kv_heads * vd].view(kv_heads, vd).to(cache.v.dtype)

    def attention(self, qkv, cache, plan, n_heads, kv_heads, head_dim, scale, window, out_dtype, store=False,
                  keep_first=0, value_dim=None, slopes=None, sinks=None):
        keep_first = keep_first or 0
        if store:
            self.kv_store(qkv, cache, plan, n_heads, kv_heads, head_dim, value_dim)
        g = cache.group_index
        vd = head_dim if value_dim is None else value_dim
        out = torch.zeros(plan.T, n_heads * vd)
        rep = n_heads // kv_heads
        for t in range(plan.T):
            s = int(plan.token_seq[t])
            if int(plan.seq_slot[s]) < 0:
                continue
            p = int(plan.positions[t])
            lo = max(0, p - window + 1) if window > 0 else 0
            pos = torch.arange(lo, p + 1)
            if window > 0 and keep_first > 0 and lo > 0:
                pos = torch.cat([torch.arange(0, min(keep_first, lo)), pos])
            pages = plan.pages[g][s, pos // PAGE].long()
            assert (pages >= 0).all(), "a position is read whose page is not held"
            k = cache.k[pages, :, pos % PAGE, :].float()      # [keys, kv_heads, hd]
            v = cache.v[pages, :, pos % PAGE, :].float()
            q = qkv[t, :n_heads * head_dim].float().view(n_heads, head_dim)
            for h in range(n_heads):
                sc = (k[:, h // rep, :] @ q[h]) * scale
                if slopes is not None:
                    sc = sc - slopes[h] * (p - pos).float()
                if sinks is not None:       # one more term of the denominator, without a value
                    pr = torch.softmax(torch.cat([sc, sinks[h:h + 1]]), 0)[:-1]
                else:
                    pr = torch.softmax(sc, 0)
                out[t, h * vd:(h + 1) * vd] = pr @ v[:, h // rep, :]
        return out.to(out_dtype)

    # ------------------------------------------------------------------ RMS norm, gates
    def rmsnorm(self, x, w, eps, out_dtype, offset=0.0):
        x = x.float()
        return (x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * (offset + w)).to(out_dtype)

    def add_normed(self, x, branches, w, eps, offset=0.0):
        total = None
        for rows, factor in branches:
            term = rows.float() * factor
            total = term if total is None else total + term
        x += self.rmsnorm(total, w, eps, torch.float32, offset)
        return x

    def gated_act(self, gu, activation, limit=0.0, alpha=1.0, shift=0.0):
        n = gu.shape[1] // 2
        g, u = gu[:, :n].float(), gu[:, n:].float()
        if activation == "silu":
            y = g * torch.sigmoid(g) * u
        else:
            g, u = g.clamp(max=limit), u.clamp(-limit, limit)
            y = g * torch.sigmoid(alpha * g) * (u + shift)
        return y.to(gu.dtype)

    # ------------------------------------------------------------------ Mamba-2
    @staticmethod
    def _sequences(plan):
        slots, starts, cu = plan.seq_slot.tolist(), plan.seq_start.tolist(), plan.cu_new.tolist()
        return [(slots[i], starts[i], cu[i], cu[i + 1]) for i in range(plan.n)]

    def conv_silu(self, proj, col0, channels, conv_w, conv_b, conv_state, plan):
        taps = conv_w.shape[1]
        out = torch.zeros(proj.shape[0], channels)
        for slot, start, t0, t1 in self._sequences(plan):
            if slot < 0:
                continue
            u = proj[t0:t1, col0:col0 + channels].float()
            if taps > 1:
                before = conv_state[slot].clone() if start > 0 else torch.zeros(taps - 1, channels)
                u = torch.cat([before, u])
                conv_state[slot] = u[-(taps - 1):]
            acc = conv_b.clone().expand(t1 - t0, channels).clone()
            for j in range(taps):
                acc += conv_w[:, j] * u[j:j + t1 - t0]
            out[t0:t1] = acc * torch.sigmoid(acc)
        return out.to(proj.dtype)

    def ssd_scan(self, xbc, proj, dt_col, dt_bias, a_log, skip, state, plan, heads, vdim, groups, n_state):
        inner, gn = heads * vdim, groups * n_state
        y = torch.zeros(xbc.shape[0], inner)
        per = heads // groups
        for slot, start, t0, t1 in self._sequences(plan):
            if slot < 0:
                continue
            S = state[slot].clone() if start > 0 else torch.zeros(heads, vdim, n_state)
            for t in range(t0, t1):
                x = xbc[t, :inner].float().view(heads, vdim)
                B = xbc[t, inner:inner + gn].float().view(groups, n_state).repeat_interleave(per, 0)
                C = xbc[t, inner + gn:inner + 2 * gn].float().view(groups, n_state).repeat_interleave(per, 0)
                dt = torch.nn.functional.softplus(proj[t, dt_col:dt_col + heads].float() + dt_bias)
                a = torch.exp(-torch.exp(a_log) * dt)
                S = a[:, None, None] * S + (dt[:, None] * x)[:, :, None] * B[:, None, :]
                y[t] = ((S * C[:, None, :]).sum(-1) + skip[:, None] * x).reshape(-1)
            state[slot] = S
        return y

    def gated_group_norm(self, y, proj, z_col, w, parts, eps, out_dtype, gate_first=True, gate="silu"):
        n = y.shape[1]
        z = proj[:, z_col:z_col + n].float()
        gate = torch.sigmoid(z) if gate == "sigmoid" else z * torch.sigmoid(z)
        g = (y * gate if gate_first else y).view(y.shape[0], parts, n // parts)
        g = (g * torch.rsqrt((g * g).mean(-1, keepdim=True) + eps)).reshape(y.shape[0], n) * w
        return (g if gate_first else g * gate).to(out_dtype)

    # ------------------------------------------------------------------ branches with norms of their own, gates
    def add_branches(self, x, branches, gain, eps):
        total = torch.zeros_like(x)
        for b in branches:
            rows = b[0].float()
            if len(b) > 2 and b[2] is not None:
                rows = rows * torch.rsqrt((rows * rows).mean(-1, keepdim=True) + eps) * b[2]
            total += b[1] * rows
        x += total if gain is None else gain * total
        return x

    def qkv_norm(self, proj, positions, heads, kv_heads, head_dim, value_dim, out_dtype, q_gain=None, k_gain=None,
                 unit_values=False, eps=0.0, temp_coef=0.0, temp_every=1):
        q_w, k_w = heads * head_dim, kv_heads * head_dim
        unit = lambda t: t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps)  # noqa: E731
        q, k = proj[:, :q_w].float(), proj[:, q_w:q_w + k_w].float()
        v = proj[:, q_w + k_w:q_w + k_w + kv_heads * value_dim].float()
        if q_gain is not None:
            q = unit(q) * q_gain
        if k_gain is not None:
            k = unit(k) * k_gain
        if temp_coef:
            q = q * (1.0 + temp_coef * torch.log(((positions.long() + 1) // temp_every + 1).float()))[:, None]
        if unit_values:
            v = unit(v.view(-1, kv_heads, value_dim)).reshape(-1, kv_heads * value_dim)
        return torch.cat([q, k, v], 1).to(out_dtype)

    def gate_mul(self, a, proj, z_col, gate="sigmoid"):
        z = proj[:, z_col:z_col + a.shape[1]].float()
        return (a.float() * (torch.sigmoid(z) if gate == "sigmoid" else z * torch.sigmoid(z))).to(a.dtype)

    # ------------------------------------------------------------------ mLSTM, minGRU
    def mlstm_gates(self, h, w, bias, heads, cap):
        g = h.float() @ w.float().t() + bias
        if cap > 0:
            g = cap * torch.tanh(g / cap)
        return torch.cat([g[:, :heads], torch.nn.functional.logsigmoid(g[:, heads:])], 1)

    def mlstm_scan(self, proj, q_col, k_col, v_col, gates, state, plan, heads, dim, vdim, floor):
        out = torch.zeros(proj.shape[0], heads * vdim)
        for slot, start, t0, t1 in self._sequences(plan):
            if slot < 0:
                continue
            fresh = start == 0
            S = torch.zeros(heads, dim, vdim) if fresh else state["S"][slot].clone()
            n = torch.zeros(heads, dim) if fresh else state["n"][slot].clone()
            m = torch.zeros(heads) if fresh else state["m"][slot].clone()
            for t in range(t0, t1):
                q = proj[t, q_col:q_col + heads * dim].float().view(heads, dim) * dim ** -0.5
                k = proj[t, k_col:k_col + heads * dim].float().view(heads, dim)
                v = proj[t, v_col:v_col + heads * vdim].float().view(heads, vdim)
                li, lf = gates[t, :heads], gates[t, heads:]
                m_new = torch.maximum(lf + m, li)
                keep, take = torch.exp(lf + m - m_new), torch.exp(li - m_new)
                S = keep[:, None, None] * S + take[:, None, None] * k[:, :, None] * v[:, None, :]
                n = keep[:, None] * n + take[:, None] * k
                m = m_new
                den = torch.maximum((n * q).sum(-1).abs(), torch.exp(-m)) + floor
                out[t] = (torch.einsum("hdv,hd->hv", S, q) / den[:, None]).reshape(-1)
            state["S"][slot], state["n"][slot], state["m"][slot] = S, n, m
        return out

    def mingru(self, proj, z_col, x_col, g_col, bias_z, bias_x, state, plan, width, out_dtype, pieces=None):
        out = torch.zeros(proj.shape[0], width)
        for slot, start, t0, t1 in self._sequences(plan):
            if slot < 0:
                continue
            S = state[slot].clone() if start > 0 else torch.zeros(width)
            for t in range(t0, t1):
                z = torch.sigmoid(proj[t, z_col:z_col + width].float() + bias_z)
                u = proj[t, x_col:x_col + width].float() + bias_x
                S = (1 - z) * S + z * torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
                g = proj[t, g_col:g_col + width].float()
                out[t] = S * g * torch.sigmoid(g)
            state[slot] = S
        return out.to(out_dtype)

    # ------------------------------------------------------------------ a table of token pairs
    def pair_table_add(self, x, plan, table, state, mul_prev, mul_cur, buckets):
        tokens = plan.tokens.tolist()
        for slot, start, t0, t1 in self._sequences(plan):
            if slot < 0:
                continue
            for t in range(t0, t1):
                if start + t - t0 == 0:
                    row = buckets
                else:
                    prev = tokens[t - 1] if t > t0 else int(state[slot, 0])
                    row = (prev * mul_prev + tokens[t] * mul_cur) % buckets
                x[t] += table[row].float()
            state[slot, 0] = tokens[t1 - 1]
        return x

    # ------------------------------------------------------------------ rotation, rows of low rank, products per head
    def rotate(self, src, dst, positions, heads, src_col, src_head, dst_col, dst_head, width, freqs, magnitude, dims):
        half = dims // 2
        a = positions.double()[:, None] * freqs.double()[None, :]
        c, s = (torch.cos(a) * magnitude).float(), (torch.sin(a) * magnitude).float()
        for h in range(heads):
            x = src[:, src_col + h * src_head: src_col + h * src_head + width].float()
            u, v = x[:, :half], x[:, half:dims]
            y = torch.cat([u * c - v * s, v * c + u * s, x[:, dims:]], 1)
            dst[:, dst_col + h * dst_head: dst_col + h * dst_head + width] = y.to(dst.dtype)
        return dst

    def latent_rows(self, down, plan, q_rank, q_norm, kv_norm, kv_rank, rot_dim, eps, rotary, cache, out_dtype):
        c_q = self.rmsnorm(down[:, :q_rank], q_norm, eps, out_dtype)
        if cache is not None:
            c = self.rmsnorm(down[:, q_rank:q_rank + kv_rank], kv_norm, eps, torch.float32)
            k_r = torch.zeros(down.shape[0], rot_dim)
            self.rotate(down, k_r, plan.positions, 1, q_rank + kv_rank, rot_dim, 0, rot_dim, rot_dim, rotary.freqs,
                        rotary.magnitude, rotary.dims)
            g = cache.group_index
            for t in range(plan.T):
                s = int(plan.token_seq[t])
                if int(plan.seq_slot[s]) < 0:
                    continue
                p = int(plan.positions[t])
                page = int(plan.pages[g][s, p // PAGE])
                assert page >= 0, "a position is written whose page is not held"
                cache.k[page, 0, p % PAGE, :] = c[t].to(cache.k.dtype)
                cache.v[page, 0, p % PAGE, :] = k_r[t].to(cache.v.dtype)
        return c_q

    def head_linear(self, a, a_col, a_head, w, out, out_col, out_head):
        heads, n, k = w.shape
        for h in range(heads):
            out[:, out_col + h * out_head: out_col + h * out_head + n] = \
                (a[:, a_col + h * a_head: a_col + h * a_head + k].float() @ w[h].float().t()).to(out.dtype)
        return out

    def latent_attention(self, rows, cache, plan, heads, kv_rank, rot_dim, scale, out_dtype):
        g = cache.group_index
        out = torch.zeros(plan.T, heads * kv_rank)
        q = rows.float().view(plan.T, heads, kv_rank + rot_dim)
        for t in range(plan.T):
            s = int(plan.token_seq[t])
            if int(plan.seq_slot[s]) < 0:
                continue
            pos = torch.arange(0, int(plan.positions[t]) + 1)
            pages = plan.pages[g][s, pos // PAGE].long()
            assert (pages >= 0).all(), "a position is read whose page is not held"
            c = cache.k[pages, 0, pos % PAGE, :].float()
            k_r = cache.v[pages, 0, pos % PAGE, :].float()
            sc = (q[t, :, :kv_rank] @ c.t() + q[t, :, kv_rank:] @ k_r.t()) * scale          # [heads, keys]
            out[t] = (torch.softmax(sc, 1) @ c).reshape(-1)
        return out.to(out_dtype)

    # ------------------------------------------------------------------ gated delta rule
    def delta_rule(self, qkv, proj, b_col, a_col, a_log, dt_bias, state, plan, heads, kv_heads, dim, vdim, unit_eps):
        qk = kv_heads * dim
        out = torch.zeros(qkv.shape[0], heads * vdim)
        per = heads // kv_heads
        for slot, start, t0, t1 in self._sequences(plan):
            if slot < 0:
                continue
            S = state[slot].clone() if start > 0 else torch.zeros(heads, dim, vdim)
            for t in range(t0, t1):
                q = qkv[t, :qk].float().view(kv_heads, dim)
                k = qkv[t, qk:2 * qk].float().view(kv_heads, dim)
                q = (q * torch.rsqrt((q * q).sum(-1, keepdim=True) + unit_eps) * dim ** -0.5).repeat_interleave(per, 0)
                k = (k * torch.rsqrt((k * k).sum(-1, keepdim=True) + unit_eps)).repeat_interleave(per, 0)
                v = qkv[t, 2 * qk:].float().view(heads, vdim)
                beta = torch.sigmoid(proj[t, b_col:b_col + heads].float())
                g = torch.exp(-torch.exp(a_log) * torch.nn.functional.softplus(proj[t, a_col:a_col + heads].float() + dt_bias))
                S = g[:, None, None] * S
                u = beta[:, None] * (v - torch.einsum("hdv,hd->hv", S, k))
                S = S + k[:, :, None] * u[:, None, :]
                out[t] = torch.einsum("hdv,hd->hv", S, q).reshape(-1)
            state[slot] = S
        return out

    # ------------------------------------------------------------------ experts by table
    def moe_route(self, tokens, T, table, experts, top):
        return table[tokens[:T].long()].long()            # [T, top]: the expert of every (token, choice) pair

    def moe_gate_up(self, h, w_gate_up, routing, out_dtype):
        T, top = routing.shape
        n = w_gate_up.shape[1] // 2
        out = torch.zeros(T * top, n)
        for t in range(T):
            for k in range(top):
                gu = w_gate_up[routing[t, k]].float() @ h[t].float()
                out[t * top + k] = gu[:n] * torch.sigmoid(gu[:n]) * gu[n:]
        return out.to(out_dtype)

    def moe_down(self, inner, w_down, routing):
        T, top = routing.shape
        out = torch.zeros(T, top, w_down.shape[1])
        for t in range(T):
            for k in range(top):
                out[t, k] = w_down[routing[t, k]].float() @ inner[t * top + k].float()
        return out

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
