"""Stand-ins for the CUDA kernels, written with torch on the CPU, for tests of the host side.

The product path has no CPU implementation.  These functions exist only so that the tests that
run without a GPU can drive the real step function, cache manager, scheduler and trace replay
and check their bookkeeping (paging, block tables, slot mapping, portions, page reuse) against
the plain implementation.  Each method restates what the kernel of the same name must do; the
GPU tests compare the kernels themselves with their plain references.
"""
from __future__ import annotations

import math

import torch


class EmulatedKernels:
    def gather_rows(self, table, ids):
        return table[ids.long()].clone()

    def late_tokens(self, token_ids, cu_seqlens, source, sampled):
        for i, j in enumerate(source.tolist()):
            if j >= 0:
                token_ids[int(cu_seqlens[i])] = sampled[j]

    def rmsnorm(self, x, gamma, eps, out_dtype=None):
        xf = x.float()
        r = 1.0 / torch.sqrt((xf * xf).mean(-1, keepdim=True) + eps)
        return (xf * r * gamma.float()).to(out_dtype or x.dtype)

    def residual_rmsnorm(self, y, gamma, eps, residual, rounded_dtype=None, keep_residual=True, next_norm=None):
        r = self.rmsnorm(y.float(), gamma, eps)
        if residual is not None:
            residual += r
            r = residual
        if next_norm is not None:
            return r, self.rmsnorm(r, *next_norm).to(rounded_dtype)
        return (r if keep_residual else None), (r.to(rounded_dtype) if rounded_dtype is not None else None)

    def stream_add(self, x, emb, table, index):
        x += table[index].float()
        if emb is not None:
            x += emb
        return x

    def polynorm(self, z, coef, eps, out_dtype=None):
        zf = z.float()
        n = lambda v: v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)
        return (coef[0] * n(zf) + coef[1] * n(zf * zf) + coef[2] * n(zf * zf * zf) + coef[3]).to(out_dtype or z.dtype)

    def softcap(self, logits, cap):
        logits.copy_(cap * torch.tanh(logits / cap))
        return logits

    def latent_prepare(self, proj, c_gamma, eps, positions, cos, sin, slot_mapping, cache_layer, num_heads, head_dim, rot_dim,
                       kv_rank, out_dtype, with_gate=True, write_kv=True, halves=False):
        T, row = proj.shape[0], kv_rank + rot_dim
        x = proj.float()
        qw = num_heads * (head_dim + rot_dim)
        pos = positions.long()

        def turn(v):          # [..., rot_dim]: pairs (2i, 2i + 1) below the tables' width
            if cos is None:
                return v
            half = cos.shape[1]
            c, s = cos[pos], sin[pos]
            while c.dim() < v.dim():
                c, s = c.unsqueeze(1), s.unsqueeze(1)
            out = v.clone()
            if halves:    # pairs (i, i + half)
                a, b = v[..., :half], v[..., half:2 * half]
                out[..., :half] = a * c - b * s
                out[..., half:2 * half] = b * c + a * s
                return out
            a, b = v[..., 0:2 * half:2], v[..., 1:2 * half:2]
            out[..., 0:2 * half:2] = a * c - b * s
            out[..., 1:2 * half:2] = b * c + a * s
            return out

        q = x[:, :qw].view(T, num_heads, head_dim + rot_dim)
        q_plain = q[:, :, :head_dim].contiguous().to(out_dtype)
        q_row = torch.zeros((T, num_heads, row), dtype=out_dtype)
        q_row[:, :, kv_rank:] = turn(q[:, :, head_dim:]).to(out_dtype)
        if write_kv:
            c = self.rmsnorm(x[:, qw:qw + kv_rank], c_gamma, eps)
            line = torch.cat([c, turn(x[:, qw + kv_rank:qw + row])], dim=1).to(out_dtype)
            ps = cache_layer.shape[3]
            for t in range(T):
                slot = int(slot_mapping[t])
                if slot >= 0:
                    cache_layer[slot // ps, 0, 0, slot % ps, :] = line[t]
        gate = torch.sigmoid(x[:, qw + row:qw + row + num_heads]) if with_gate else None
        return q_plain, q_row, gate

    def head_linear(self, x, weight, out=None, out_dtype=None):
        y = torch.einsum("thk,hnk->thn", x.float(), weight.float()).contiguous()
        if out is None:
            return y.to(out_dtype or x.dtype)
        out.copy_(y.to(out.dtype))
        return out

    def latent_attention(self, q_row, cache_layer, meta, num_heads, row, value_dim, scale, gate=None, sinks=None):
        T = q_row.shape[0]
        ps = cache_layer.shape[3]
        out = torch.zeros((T, num_heads, value_dim), dtype=q_row.dtype)
        cu = meta.cu_seqlens.tolist()
        for s in range(meta.num_seqs):
            ctx = int(meta.ctx_lens[s])
            if ctx <= 0:
                continue
            q_len = cu[s + 1] - cu[s]
            table = meta.block_tables[s].tolist()
            for i in range(q_len):
                t, pos = cu[s] + i, ctx - q_len + i
                pages = [table[j // ps] for j in range(pos + 1)]
                assert all(p >= 0 for p in pages), "attention reads a page that was given back"
                rows = cache_layer[pages, 0, 0, [j % ps for j in range(pos + 1)], :].float()
                sc = (q_row[t].float() @ rows.T) * scale                            # [heads, keys]
                if sinks is not None:
                    p = torch.softmax(torch.cat([sc, sinks.float()[:, None]], dim=1), -1)[:, :-1]
                else:
                    p = torch.softmax(sc, -1)
                o = p @ rows[:, :value_dim]
                if gate is not None:
                    o = o * gate[t][:, None]
                out[t] = o.to(q_row.dtype)
        return out

    def moe_experts(self, x, chosen, gate_up, down, weight, add=None, out_dtype=None, weights=None, activation="silu"):
        T, ff = x.shape[0], gate_up.shape[1] // 2
        out = torch.zeros((T, x.shape[1])) if add is None else add.clone().float()
        for t in range(T):
            for j, e in enumerate(chosen[t].tolist()):
                gu = gate_up[e].float() @ x[t].float()
                if activation == "relu2":         # plain experts: every row of the first matrix is an up row
                    a = torch.relu(gu) ** 2
                else:
                    g, u = gu[:ff], gu[ff:]
                    a = g / (1.0 + torch.exp(-g)) * u
                w = weight * (float(weights[t, j]) if weights is not None else 1.0)
                out[t] += w * (down[e].float() @ a.to(x.dtype).float())
        return out.to(out_dtype or x.dtype)

    # ---- the kernels of the Dynamic-Tanh norms, the unit-norm attention, the mLSTM and the routed experts
    def dynamic_tanh(self, x, alpha, weight, bias, out_dtype=None):
        return (torch.tanh(alpha * x.float()) * weight + bias).to(out_dtype or x.dtype)

    def residual_dynamic_tanh(self, y, norm, x, next_norm, out_dtype):
        x += self.dynamic_tanh(y.float(), *norm)
        return x, (self.dynamic_tanh(x, *next_norm, out_dtype=out_dtype) if next_norm is not None else None)

    def scale_rows(self, x, scale):
        return x.float() * scale

    def act_rows(self, u, activation, out_dtype, row_scale=None):
        assert activation == "relu2"
        a = torch.relu(u.float()) ** 2
        if row_scale is not None:
            a = a * row_scale[:, None]
        return a.to(out_dtype)

    def moe_route_top(self, scores, correction, experts, top, groups, keep, weight_eps, shared_gate=False):
        s = torch.sigmoid(scores[:, :experts].float())
        c = s + correction
        per = experts // groups
        gs = c.view(-1, groups, per).topk(min(2, per), dim=-1).values.sum(-1)
        kept = gs.topk(keep, dim=-1).indices
        allowed = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, kept, True).repeat_interleave(per, dim=1)
        chosen = c.masked_fill(~allowed, float("-inf")).topk(top, dim=-1).indices
        w = s.gather(1, chosen)
        w = w / (w.sum(-1, keepdim=True) + weight_eps)
        gate = torch.sigmoid(scores[:, experts].float()) if shared_gate else None
        return chosen.to(torch.int32), w, gate

    def qk_unit_prepare(self, proj, eps, positions, cos, sin, slot_mapping, cache_layer, num_heads, num_kv_heads, head_dim,
                        value_dim, slot_dim, out_dtype, halves=False, with_gate=True, write_kv=True):
        T = proj.shape[0]
        x = proj.float()
        pos = positions.long()

        def turn(v):           # [T, heads, head_dim]
            if cos is None:
                return v
            half = cos.shape[1]
            c, s = cos[pos][:, None, :], sin[pos][:, None, :]
            out = v.clone()
            if halves:
                a, b = v[..., :half], v[..., half:2 * half]
                out[..., :half], out[..., half:2 * half] = a * c - b * s, b * c + a * s
            else:
                a, b = v[..., 0:2 * half:2], v[..., 1:2 * half:2]
                out[..., 0:2 * half:2], out[..., 1:2 * half:2] = a * c - b * s, b * c + a * s
            return out

        unit = lambda v: v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)
        qw = num_heads * head_dim
        q = torch.zeros((T, num_heads, slot_dim))
        q[:, :, :head_dim] = unit(turn(x[:, :qw].view(T, num_heads, head_dim)))
        col = qw
        if write_kv:
            kw, vw = num_kv_heads * head_dim, num_kv_heads * value_dim
            k = unit(turn(x[:, col:col + kw].view(T, num_kv_heads, head_dim)))
            v = x[:, col + kw:col + kw + vw].view(T, num_kv_heads, value_dim)
            col += kw + vw
            ps = cache_layer.shape[3]
            for t, slot in enumerate(slot_mapping.tolist()):
                if slot < 0:
                    continue
                cache_layer[slot // ps, 0, :, slot % ps, :] = 0
                cache_layer[slot // ps, 1, :, slot % ps, :] = 0
                cache_layer[slot // ps, 0, :, slot % ps, :head_dim] = k[t].to(cache_layer.dtype)
                cache_layer[slot // ps, 1, :, slot % ps, :value_dim] = v[t].to(cache_layer.dtype)
        gate = torch.sigmoid(x[:, col:col + num_heads]) if with_gate else None
        return q.view(T, num_heads * slot_dim).to(out_dtype), gate

    def mlstm_scan(self, proj, i_col0, f_col0, i_bias, f_bias, cu_seqlens, state_slots, state, heads, head_dim, value_dim, cap):
        T = proj.shape[0]
        D, V = head_dim, value_dim
        x = proj.float()
        q = x[:, :heads * D].view(T, heads, D) * D ** -0.5
        k = x[:, heads * D:2 * heads * D].view(T, heads, D)
        v = torch.cat([x[:, 2 * heads * D:2 * heads * D + heads * V].view(T, heads, V), torch.ones((T, heads, 1))], dim=-1)
        gi = cap * torch.tanh((x[:, i_col0:i_col0 + heads] + i_bias) / cap)
        gf = torch.nn.functional.logsigmoid(cap * torch.tanh((x[:, f_col0:f_col0 + heads] + f_bias) / cap))
        raw = torch.zeros((T, heads, V + 1))
        top = torch.zeros((T, heads))
        cu = cu_seqlens.tolist()
        for s, slot in enumerate(state_slots.tolist()):
            if slot < 0:
                continue
            S = state[slot, :heads * D * (V + 1)].view(heads, D, V + 1)
            m = state[slot, heads * D * (V + 1):heads * D * (V + 1) + heads].clone()
            for t in range(cu[s], cu[s + 1]):
                new = torch.maximum(gf[t] + m, gi[t])
                a, b = torch.exp(gf[t] + m - new), torch.exp(gi[t] - new)
                S.copy_(a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :])
                m = new                      # (the state row keeps the old m until `mlstm_output` stores the last one)
                raw[t] = torch.einsum("hdv,hd->hv", S, q[t])
                top[t] = new
        return raw.view(T, heads * (V + 1)), top

    def mlstm_output(self, raw, top, gamma, eps, den_eps, proj, g_col0, heads, head_dim, value_dim, out_dtype, token_seq, cu_seqlens,
                     state_slots, state):
        T, V = raw.shape[0], value_dim
        cu = cu_seqlens.tolist()
        for s, slot in enumerate(state_slots.tolist()):
            if slot >= 0 and cu[s + 1] > cu[s]:
                at = heads * head_dim * (V + 1)
                state[slot, at:at + heads] = top[cu[s + 1] - 1]
        r = raw.view(T, heads, V + 1)
        o = r[:, :, :V] / (torch.maximum(r[:, :, V:].abs(), torch.exp(-top)[:, :, None]) + den_eps)
        o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps)
        z = proj[:, g_col0:g_col0 + heads * V].float()
        return (o.reshape(T, heads * V) * gamma.float() * torch.sigmoid(z)).to(out_dtype)

    def act_mul(self, gate_up, activation, out_dtype=None, limit=None, alpha=None):
        inter = gate_up.shape[1] // 2
        g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
        if activation == "swiglu_clamp":
            g, u = torch.clamp(g, max=limit), torch.clamp(u, min=-limit, max=limit)
            return (g * torch.sigmoid(alpha * g) * (u + 1.0)).to(out_dtype or gate_up.dtype)
        if activation == "silu":
            a = g / (1.0 + torch.exp(-g))
        else:
            a = 0.5 * g * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (g + 0.044715 * g ** 3)))
        return (a * u).to(out_dtype or gate_up.dtype)

    def gate_up_act(self, x, weight, activation="silu", norm=None):
        return self.act_mul(self.linear(x, weight, out_dtype=torch.float32, norm=norm), activation, x.dtype)

    def qk_norm_rope_cache_write(self, proj, q_gamma, k_gamma, eps, positions, cos, sin, slot_mapping, cache_layer,
                                 num_heads, num_kv_heads, head_dim, out_dtype, with_gate=False, write_kv=True):
        T = proj.shape[0]
        qw, kw = num_heads * head_dim, num_kv_heads * head_dim
        x = proj.float()
        q = self.rmsnorm(x[:, :qw], q_gamma, eps)
        kraw = x[:, qw:qw + kw]
        kn = self.rmsnorm(kraw, k_gamma, eps)
        stacked = torch.cat([q, kn, kraw], dim=1)         # the rotation below leaves the third part alone
        qo = self.rope_cache_write(stacked, None, positions, cos, sin, slot_mapping, cache_layer, num_heads, num_kv_heads,
                                   head_dim, write_kv=write_kv, out_dtype=out_dtype) if write_kv else \
            self.rope_cache_write(q.contiguous(), None, positions, cos, sin, None, None, num_heads, num_kv_heads, head_dim,
                                  write_kv=False, out_dtype=out_dtype)
        gate = torch.sigmoid(x[:, qw + kw:]) if with_gate else None
        return qo, gate

    def causal_conv_silu(self, proj, col0, channels, weight, bias, token_seq, cu_seqlens, state_slots, state, conv_off, out_dtype):
        taps = weight.shape[1]
        u = proj[:, col0:col0 + channels].float()
        out = torch.zeros_like(u)
        cu = cu_seqlens.tolist()
        for s, slot in enumerate(state_slots.tolist()):
            if slot < 0:
                continue
            hist = state[slot, conv_off:conv_off + (taps - 1) * channels].view(taps - 1, channels)
            seq = torch.cat([hist, u[cu[s]:cu[s + 1]]], dim=0)
            n = cu[s + 1] - cu[s]
            acc = torch.zeros((n, channels))
            for j in range(taps):
                acc = acc + seq[j:j + n] * weight[:, j].float()[None, :]
            if bias is not None:
                acc = acc + bias.float()[None, :]
            out[cu[s]:cu[s + 1]] = acc / (1.0 + torch.exp(-acc))
            hist.copy_(seq[n:n + taps - 1].clone())
        return out.to(out_dtype)

    def ssm_scan(self, xbc, proj, dt_col0, dt_bias, a_log, d_skip, cu_seqlens, state_slots, state, heads, head_dim,
                 state_size, groups, columns=0, max_q_len=None, segment_tokens=None):
        T = xbc.shape[0]
        inner, P, N = heads * head_dim, head_dim, state_size
        xf = xbc.float()
        y = torch.zeros((T, inner))
        cu = cu_seqlens.tolist()
        for s, slot in enumerate(state_slots.tolist()):
            if slot < 0:
                continue
            S = state[slot, :heads * N * P].view(heads, N, P)
            for t in range(cu[s], cu[s + 1]):
                dt = torch.nn.functional.softplus(proj[t, dt_col0:dt_col0 + heads].float() + dt_bias.float(), threshold=20.0)
                for h in range(heads):
                    g = h // (heads // groups)
                    x = xf[t, h * P:(h + 1) * P]
                    B = xf[t, inner + g * N:inner + (g + 1) * N]
                    C = xf[t, inner + groups * N + g * N:inner + groups * N + (g + 1) * N]
                    S[h] = torch.exp(-torch.exp(a_log[h].float()) * dt[h]) * S[h] + dt[h] * B[:, None] * x[None, :]
                    y[t, h * P:(h + 1) * P] = S[h].t() @ C + d_skip[h].float() * x
        return y

    def gated_group_rmsnorm(self, y, proj, gamma, eps, parts, out_dtype):
        rows, width = y.shape
        z = proj[:, :width].float()
        v = (y * (z / (1.0 + torch.exp(-z)))).view(rows, parts, width // parts)
        v = v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)
        return (v.reshape(rows, width) * gamma.float()).to(out_dtype)

    def silu_mul(self, gate_up):
        inter = gate_up.shape[1] // 2
        g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
        return (g / (1.0 + torch.exp(-g)) * u).to(gate_up.dtype)

    def rope_cache_write(self, qkv, bias, positions, cos, sin, slot_mapping, cache_layer,
                         num_heads, num_kv_heads, head_dim, write_kv=True, out_dtype=None):
        out_dtype = out_dtype or qkv.dtype
        T = qkv.shape[0]
        x = qkv.float()
        if bias is not None:
            x = x + bias.float()
        pos = positions.long()

        def rot(t):   # [T, heads, hd]; the tables' width says how much of a head is rotated
            if cos is None:
                return t
            half = cos.shape[1]
            c, s = cos[pos][:, None, :], sin[pos][:, None, :]
            a, b, rest = t[..., :half], t[..., half:2 * half], t[..., 2 * half:]
            return torch.cat([a * c - b * s, a * s + b * c, rest], -1)

        q_dim, kv_dim = num_heads * head_dim, num_kv_heads * head_dim
        q = rot(x[:, :q_dim].view(T, num_heads, head_dim))
        if write_kv:
            k = rot(x[:, q_dim:q_dim + kv_dim].view(T, num_kv_heads, head_dim)).to(out_dtype)
            v = x[:, q_dim + kv_dim:].view(T, num_kv_heads, head_dim).to(out_dtype)
            ps = cache_layer.shape[3]
            for t in range(T):
                slot = int(slot_mapping[t])
                if slot < 0:
                    continue
                cache_layer[slot // ps, 0, :, slot % ps, :] = k[t]
                cache_layer[slot // ps, 1, :, slot % ps, :] = v[t]
        return q.reshape(T, q_dim).to(out_dtype)

    def qkv_rope_cache_write(self, x, weight, bias, positions, cos, sin, slot_mapping, cache_layer,
                             num_heads, num_kv_heads, head_dim, norm=None):
        return self.rope_cache_write(self.linear(x, weight, norm=norm), bias, positions, cos, sin, slot_mapping, cache_layer,
                                     num_heads, num_kv_heads, head_dim)

    def paged_attention(self, q, cache_layer, meta, num_heads, num_kv_heads, head_dim, scale, window,
                        softcap=None, sinks=None, gate=None):
        T = q.shape[0]
        ps = cache_layer.shape[3]
        out = torch.zeros_like(q).view(T, num_heads, head_dim)
        qv = q.view(T, num_heads, head_dim).float()
        cu = meta.cu_seqlens.tolist()
        for s in range(meta.num_seqs):
            ctx = int(meta.ctx_lens[s])
            if ctx <= 0:
                continue
            q_len = cu[s + 1] - cu[s]
            table = meta.block_tables[s].tolist()
            for i in range(q_len):
                t = cu[s] + i
                pos = ctx - q_len + i
                lo = max(0, pos - window + 1) if window else 0
                keys = list(range(lo, pos + 1))
                pages = [table[j // ps] for j in keys]
                assert all(p >= 0 for p in pages), "attention reads a page that was given back"
                offs = [j % ps for j in keys]
                for h in range(num_heads):
                    g = h * num_kv_heads // num_heads
                    K = cache_layer[pages, 0, g, offs, :].float()
                    V = cache_layer[pages, 1, g, offs, :].float()
                    sc = (K @ qv[t, h]) * scale
                    if softcap is not None:
                        sc = softcap * torch.tanh(sc / softcap)
                    if sinks is not None:
                        p = torch.softmax(torch.cat([sc, sinks[h:h + 1].float()]), 0)[:-1]
                    else:
                        p = torch.softmax(sc, 0)
                    o = p @ V
                    if gate is not None:
                        o = o * gate[t, h]
                    out[t, h] = o.to(q.dtype)
        return out.view(T, num_heads * head_dim)

    # ---- the kernels of the pre-norm stream block, the mamba1 mixer, the attention that mixes its weights across heads
    # ---- and the gated delta rule
    def scale_add_sinusoid(self, x, positions, frequencies, scale):
        ang = positions.double()[:, None] * frequencies.double()[None, :]
        pe = torch.stack([torch.sin(ang), torch.cos(ang)], dim=-1).reshape(x.shape[0], -1)[:, :x.shape[1]]
        return (x.double() * scale + pe).float()

    def stream_add_norm(self, x, y, norm, out_dtype):
        if y is not None:
            x += y
        if out_dtype is None:
            return x, None
        if norm is None:
            return x, x.to(out_dtype)
        return x, self.rmsnorm(x, norm[0], norm[1]).to(out_dtype)

    def gelu_mul_columns(self, g, table_rows, col0, out_dtype):
        gf = g.float()
        a = 0.5 * gf * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (gf + 0.044715 * gf ** 3)))
        return (a * table_rows[:, col0:col0 + g.shape[1]].float()).to(out_dtype)

    def column_slice(self, x, col0, n, out_dtype):
        return x[:, col0:col0 + n].to(out_dtype).contiguous()

    def scaled_sum(self, a, sa, b, sb):
        if a is None:
            return b.float() * sb
        a.mul_(sa).add_(b.float() * sb)
        return a

    def selective_scan(self, u, dt_raw, dt_bias, a, bc, b_col0, c_col0, d_skip, z, z_col0, cu_seqlens, state_slots, state, out_dtype):
        T, inner = u.shape
        N = a.shape[1]
        uf = u.float()
        y = torch.zeros((T, inner))
        cu = cu_seqlens.tolist()
        for s, slot in enumerate(state_slots.tolist()):
            if slot < 0:
                continue
            S = state[slot, :inner * N].view(inner, N)
            for t in range(cu[s], cu[s + 1]):
                dt = torch.nn.functional.softplus(dt_raw[t].float() + dt_bias, threshold=20.0)
                B, C = bc[t, b_col0:b_col0 + N].float(), bc[t, c_col0:c_col0 + N].float()
                S.copy_(torch.exp(dt[:, None] * a) * S + (dt * uf[t])[:, None] * B[None, :])
                y[t] = S @ C + d_skip * uf[t]
        zf = z[:, z_col0:z_col0 + inner].float()
        return (y * zf / (1.0 + torch.exp(-zf))).to(out_dtype)

    @staticmethod
    def _kv_planes(cache_layer, G, ps, d, vd):
        """Views [pages, G, page, d] and [pages, G, page, vd] of a cache layer in either layout."""
        flat = cache_layer.reshape(cache_layer.shape[0], -1)
        nk = G * ps * d
        return flat[:, :nk].view(-1, G, ps, d), flat[:, nk:nk + G * ps * vd].view(-1, G, ps, vd)

    def kv_prepare(self, proj, slot_mapping, cache_layer, num_heads, num_kv_heads, head_dim, value_dim, value_norm_eps, out_dtype,
                   write_kv=True):
        T = proj.shape[0]
        qw, kw = num_heads * head_dim, num_kv_heads * head_dim
        x = proj.float()
        if write_kv:
            ps = cache_layer.numel() // cache_layer.shape[0] // (num_kv_heads * (head_dim + value_dim))
            K, V = self._kv_planes(cache_layer, num_kv_heads, ps, head_dim, value_dim)
            k = x[:, qw:qw + kw].view(T, num_kv_heads, head_dim)
            v = x[:, qw + kw:].view(T, num_kv_heads, value_dim)
            if value_norm_eps is not None:
                v = v / torch.sqrt((v * v).mean(-1, keepdim=True) + value_norm_eps)
            for t, slot in enumerate(slot_mapping.tolist()):
                if slot < 0:
                    continue
                K[slot // ps, :, slot % ps] = k[t].to(cache_layer.dtype)
                V[slot // ps, :, slot % ps] = v[t].to(cache_layer.dtype)
        return x[:, :qw].to(out_dtype).contiguous()

    def talking_attention(self, q, cache_layer, meta, positions, num_heads, num_kv_heads, head_dim, value_dim, scale, r1, r2,
                          talk, chunk):
        T = q.shape[0]
        ps = meta.page_size
        K, V = self._kv_planes(cache_layer, num_kv_heads, ps, head_dim, value_dim)
        out = torch.zeros((T, num_heads, value_dim))
        qv = q.view(T, num_heads, head_dim).float()
        cu = meta.cu_seqlens.tolist()
        rep = num_heads // num_kv_heads
        for s in range(meta.num_seqs):
            ctx = int(meta.ctx_lens[s])
            if ctx <= 0:
                continue
            q_len = cu[s + 1] - cu[s]
            table = meta.block_tables[s].tolist()
            for i in range(q_len):
                t = cu[s] + i
                pos = ctx - q_len + i
                assert pos == int(positions[t])
                lo = (pos // chunk) * chunk if chunk else 0
                keys = list(range(lo, pos + 1))
                pages = [table[j // ps] for j in keys]
                assert all(p >= 0 for p in pages), "attention reads a page that was given back"
                offs = [j % ps for j in keys]
                dist = torch.tensor([pos - j for j in keys], dtype=torch.float32)
                P = torch.zeros((num_heads, len(keys)))
                for h in range(num_heads):
                    sc = (K[pages, h // rep, offs, :].float() @ qv[t, h]) * scale
                    if r1 is not None:
                        sc = sc - r1[h] * torch.log1p(r2[h] * dist)
                    P[h] = torch.softmax(sc, 0)
                if talk is not None:
                    P = talk.float() @ P
                for h in range(num_heads):
                    out[t, h] = P[h] @ V[pages, h // rep, offs, :].float()
        return out.view(T, num_heads * value_dim).to(q.dtype)

    def delta_rule(self, qkv, proj, b_col0, a_col0, a_log, dt_bias, cu_seqlens, state_slots, state, heads, qk_heads, head_dim,
                   value_dim, unit_eps):
        T = qkv.shape[0]
        qk = qk_heads * head_dim
        x = qkv.float()
        q = x[:, :qk].view(T, qk_heads, head_dim)
        k = x[:, qk:2 * qk].view(T, qk_heads, head_dim)
        v = x[:, 2 * qk:].view(T, heads, value_dim)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + unit_eps) * head_dim ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + unit_eps)
        rep = heads // qk_heads
        beta = torch.sigmoid(proj[:, b_col0:b_col0 + heads].float())
        g = torch.exp(-torch.exp(a_log) * torch.nn.functional.softplus(proj[:, a_col0:a_col0 + heads].float() + dt_bias, threshold=20.0))
        o = torch.zeros((T, heads, value_dim))
        cu = cu_seqlens.tolist()
        for s, slot in enumerate(state_slots.tolist()):
            if slot < 0:
                continue
            S = state[slot, :heads * head_dim * value_dim].view(heads, head_dim, value_dim)
            for t in range(cu[s], cu[s + 1]):
                for h in range(heads):
                    kh, qh = k[t, h // rep], q[t, h // rep]
                    Sh = g[t, h] * S[h]
                    u = beta[t, h] * (v[t, h] - Sh.t() @ kh)
                    Sh = Sh + kh[:, None] * u[None, :]
                    S[h] = Sh
                    o[t, h] = Sh.t() @ qh
        return o.view(T, heads * value_dim)

    def head_norm_gate(self, o, gamma, eps, proj, g_col0, heads, value_dim, out_dtype):
        T = o.shape[0]
        of = o.float().view(T, heads, value_dim)
        of = of / torch.sqrt((of * of).mean(-1, keepdim=True) + eps) * gamma.float()
        z = proj[:, g_col0:g_col0 + heads * value_dim].float().view(T, heads, value_dim)
        return (of * z / (1.0 + torch.exp(-z))).reshape(T, heads * value_dim).to(out_dtype)

    def linear(self, x, weight, bias=None, residual=None, out_dtype=None, norm=None):
        if norm is not None:
            x = self.rmsnorm(x, *norm)
        y = x.float() @ weight.float().t()
        if bias is not None:
            y = y + bias.float()
        if residual is not None:
            y = y + residual.float()
        return y.to(out_dtype or x.dtype)

    def gate_up_silu(self, x, weight, norm=None):
        return self.silu_mul(self.linear(x, weight, norm=norm))

    def sample(self, logits, temperature=None, top_k=None, top_p=None, seeds=None, draw_index=None):
        from plain_impl import sample as plain_sample
        out = []
        for r in range(logits.shape[0]):
            T = float(temperature[r]) if temperature is not None else 0.0
            k = int(top_k[r]) if top_k is not None else 0
            p = float(top_p[r]) if top_p is not None else 1.0
            tok, _ = plain_sample(logits[r], T, int(seeds[r]) if seeds is not None else 0,
                                  int(draw_index[r]) if draw_index is not None else 0, k, p)
            out.append(tok)
        return torch.tensor(out, dtype=torch.int32)
