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
                  keep_first=0, value_dim=None, slopes=None, sinks=None, chunk=0, head_scales=None, head_scales_positive=True):
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
            if chunk > 0:
                lo = p // chunk * chunk
            pos = torch.arange(lo, p + 1)
            if window > 0 and keep_first > 0 and lo > 0:
                pos = torch.cat([torch.arange(0, min(keep_first, lo)), pos])
            pages = plan.pages[g][s, pos // PAGE].long()
            assert (pages >= 0).all(), "a position is read whose page is not held"
            k = cache.k[pages, :, pos % PAGE, :].float()      # [keys, kv_heads, hd]
            v = cache.v[pages, :, pos % PAGE, :].float()
            q = qkv[t, :n_heads * head_dim].float().view(n_heads, head_dim)
            for h in range(n_heads):
                sc = (k[:, h // rep, :] @ q[h]) * scale * (1.0 if head_scales is None else float(head_scales[h]))
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

    def conv_silu(self, proj, col0, channels, conv_w, conv_b, conv_state, plan, act="silu"):
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
            out[t0:t1] = acc * torch.sigmoid(acc) if act == "silu" else acc
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
    def rotate(self, src, dst, positions, heads, src_col, src_head, dst_col, dst_head, width, freqs, magnitude, dims,
               interleaved=False):
        half = dims // 2
        a = positions.double()[:, None] * freqs.double()[None, :]
        c, s = (torch.cos(a) * magnitude).float(), (torch.sin(a) * magnitude).float()
        for h in range(heads):
            x = src[:, src_col + h * src_head: src_col + h * src_head + width].float()
            if interleaved:
                u, v = x[:, 0:dims:2], x[:, 1:dims:2]
                y = x.clone()
                y[:, 0:dims:2], y[:, 1:dims:2] = u * c - v * s, v * c + u * s
            else:
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
        if tokens is None:                                # the table's row t is token t's choice
            return table[:T].long()
        return table[tokens[:T].long()].long()            # [T, top]: the expert of every (token, choice) pair

    def moe_pick(self, logits, correction, experts, top, groups, keep_groups, route_scale):
        s = torch.sigmoid(logits[:, :experts].float())
        choice = s + correction
        per = experts // groups
        if groups > 1:
            grouped = choice.view(-1, groups, per)
            score = grouped.topk(min(2, per), dim=-1).values.sum(-1)
            kept = score.topk(keep_groups, dim=-1).indices
            allowed = torch.zeros_like(score, dtype=torch.bool).scatter_(1, kept, True)
            choice = torch.where(allowed.repeat_interleave(per, dim=1), choice, torch.full_like(choice, -float("inf")))
        chosen = choice.topk(top, dim=-1).indices
        w = s.gather(1, chosen)
        return chosen.to(torch.int32), w / (w.sum(-1, keepdim=True) + 1e-20) * route_scale

    def moe_combine(self, x, y, weights, shared, logits, gate_col):
        out = x + (y * weights[:, :, None]).sum(1)
        if shared is not None:
            out = out + (shared if logits is None else shared * torch.sigmoid(logits[:, gate_col:gate_col + 1].float()))
        return out

    def moe_gate_up(self, h, w_gate_up, routing, out_dtype, limit=0.0, alpha=1.0, shift=0.0):
        T, top = routing.shape
        n = w_gate_up.shape[1] // 2
        out = torch.zeros(T * top, n)
        for t in range(T):
            for k in range(top):
                gu = w_gate_up[routing[t, k]].float() @ h[t].float()
                g, u = gu[:n], gu[n:]
                if limit > 0:
                    g, u = g.clamp(max=limit), u.clamp(-limit, limit)
                    out[t * top + k] = g * torch.sigmoid(alpha * g) * (u + shift)
                else:
                    out[t * top + k] = g * torch.sigmoid(g) * u
        return out.to(out_dtype)

    # ------------------------------------------------------------------ token shift, linear attention, the generalized delta rule
    def token_shift(self, h, mu, state, plan):
        out = torch.zeros_like(h, dtype=torch.float32)
        for slot, start, t0, t1 in self._sequences(plan):
            if slot < 0:
                continue
            rows = h[t0:t1].float()
            before = state[slot].clone() if start > 0 else torch.zeros_like(rows[0])
            prev = torch.cat([before[None], rows[:-1]])
            out[t0:t1] = rows + (prev - rows) * mu
            state[slot] = rows[-1]
        return out.to(h.dtype)

    def low_rank_out(self, proj, col, w2, bias, act):
        lr = proj[:, col:col + w2.shape[0]].float()       # (w2 is [rank, outputs])
        if act == "tanh":
            lr = torch.tanh(lr)
        return lr @ w2 + bias

    def gla_scan(self, proj, q_col, k_col, v_col, z, tau, state, plan, heads, dim, vdim):
        out = torch.zeros(proj.shape[0], heads * vdim)
        alpha = torch.exp(torch.nn.functional.logsigmoid(z.float()) / tau)
        for slot, start, t0, t1 in self._sequences(plan):
            if slot < 0:
                continue
            S = state[slot].clone() if start > 0 else torch.zeros(heads, dim, vdim)
            for t in range(t0, t1):
                q = proj[t, q_col:q_col + heads * dim].float().view(heads, dim) * dim ** -0.5
                k = proj[t, k_col:k_col + heads * dim].float().view(heads, dim)
                v = proj[t, v_col:v_col + heads * vdim].float().view(heads, vdim)
                S = alpha[t].view(heads, dim)[:, :, None] * S + k[:, :, None] * v[:, None, :]
                out[t] = torch.einsum("hdv,hd->hv", S, q).reshape(-1)
            state[slot] = S
        return out

    def generalized_delta_rule(self, proj, r_col, k_col, v_col, a_col, a_bias, wz, decay_coef, state, plan, heads, dim, unit_eps):
        m = heads * dim
        out = torch.zeros(proj.shape[0], m)
        w_all = torch.exp(-decay_coef * torch.sigmoid(wz.float()))
        for slot, start, t0, t1 in self._sequences(plan):
            if slot < 0:
                continue
            S = state[slot].clone() if start > 0 else torch.zeros(heads, dim, dim)
            for t in range(t0, t1):
                r, k, v = (proj[t, c:c + m].float().view(heads, dim) for c in (r_col, k_col, v_col))
                a = torch.sigmoid(proj[t, a_col:a_col + m].float() + a_bias).view(heads, dim)
                u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + unit_eps)
                uS = torch.einsum("hd,hdv->hv", u, S)
                S = w_all[t].view(heads, dim)[:, :, None] * S - (a * u)[:, :, None] * uS[:, None, :] + k[:, :, None] * v[:, None, :]
                out[t] = torch.einsum("hdv,hd->hv", S, r).reshape(-1)
            state[slot] = S
        return out

    def side_input(self, x, plan, table, col, dim, w_gate, w_proj, w_norm, eps):
        e = table[plan.tokens[:x.shape[0]].long(), col:col + dim].float()
        z = x.float() @ w_gate.float().t()
        g = 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3))) * e
        y = g @ w_proj.float().t()
        return x + y * torch.rsqrt((y * y).mean(-1, keepdim=True) + eps) * w_norm

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
