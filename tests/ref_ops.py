"""Plain PyTorch versions of every kernel, with the kernels' own signatures.

Two uses: each CUDA kernel is compared with the function of the same name here, and tests
that exercise the engine's logic without a GPU (cache, step function, scheduler) run the
engine on these instead of the CUDA kernels.  Nothing in the package imports this file.
All arithmetic is 32-bit; results are rounded once to the output's dtype.
"""

from __future__ import annotations

import torch


class RefOps:
    name = "torch-reference"

    def embedding(self, table, ids, out, scale=1.0):
        out.copy_(table[ids.long()].float() * scale)

    @staticmethod
    def _added(h, delta, rows, delta_scale):
        if delta is not None and delta.dim() == 3:  # the parts of a split matrix product
            delta = delta.sum(0)
        if rows is None:
            if delta is not None:
                h.add_(delta * delta_scale)
            return h
        x = h[rows.long()]
        if delta is not None:
            x = x + delta[rows.long()] * delta_scale
        return x

    def rmsnorm(self, h, delta, weight, eps, out, rows=None, delta_scale=1.0):
        x = self._added(h, delta, rows, delta_scale)
        normed = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
        out.copy_((weight * normed).to(out.dtype))

    def layernorm(self, h, delta, weight, eps, out, rows=None, delta_scale=1.0):
        x = self._added(h, delta, rows, delta_scale)
        centred = x - x.mean(-1, keepdim=True)
        out.copy_((centred * torch.rsqrt(centred.pow(2).mean(-1, keepdim=True) + eps) * weight).to(out.dtype))

    def add_position_rows(self, h, table, positions):
        h.add_(table[positions.long()].float())

    def relu_squared(self, x, out):
        out.copy_(torch.relu(x.float()).pow(2).to(out.dtype))

    def scale_(self, t, factor):
        t.mul_(factor)

    def scale_softcap_(self, t, factor, cap):
        t.copy_(cap * torch.tanh(t * factor / cap))

    # --- latent attention ---------------------------------------------------------------------

    def latent_prep(self, proj, positions, table, rot_dims, norm_w, eps, q_plain, q_abs, gate, cache,
                    slot_mapping, heads, dim, rot_dim, rank, page_size):
        n = proj.shape[0]
        row = rank + rot_dim
        q = proj[:, : heads * (dim + rot_dim)].reshape(n, heads, dim + rot_dim).float()
        dkv = proj[:, heads * (dim + rot_dim): heads * (dim + rot_dim) + row].float()
        g = proj[:, heads * (dim + rot_dim) + row:].float()

        def rot(x):  # [n, ..., rot_dim]
            if table is None or rot_dims == 0:
                return x
            cos, sin = table[positions.long(), 0], table[positions.long(), 1]  # [n, rot_dims/2]
            while cos.dim() < x.dim():
                cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
            out = x.clone()
            u, v = x[..., 0:rot_dims:2], x[..., 1:rot_dims:2]
            out[..., 0:rot_dims:2] = u * cos - v * sin
            out[..., 1:rot_dims:2] = v * cos + u * sin
            return out

        q_plain.copy_(q[..., :dim].reshape(n, heads * dim).to(q_plain.dtype))
        q_abs.view(n, heads, row)[:, :, rank:] = rot(q[..., dim:]).to(q_abs.dtype)
        gate.copy_(torch.sigmoid(g))
        if slot_mapping is not None:
            c = dkv[:, :rank]
            c = c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + eps) * norm_w
            rows = torch.cat([c, rot(dkv[:, rank:])], dim=-1).to(cache.dtype)
            slots = slot_mapping.long()
            cache[slots // page_size, 0, slots % page_size] = rows

    def headwise_linear(self, x, w, out, row_scale=None):
        y = torch.einsum("nhk,hok->nho", x.float(), w.float())
        if row_scale is not None:
            y = y * row_scale[..., None]
        out.copy_(y.to(out.dtype))

    # --- delta rule ---------------------------------------------------------------------------

    def delta_prep(self, qkvb, a, conv_w, A_log, dt_bias, state, slots, ctx, q_out, k_out, v_out, beta,
                   decay, heads, kv_heads, dim, vdim, taps):
        channels = conv_w.shape[0]
        matrix = heads * dim * vdim
        qk = kv_heads * dim
        slot_list = slots.tolist()
        for start, n, slot in zip(ctx.q_starts, ctx.q_lens, slot_list):
            if n == 0:
                continue
            tail = state[slot, matrix:].view(taps - 1, channels)
            x = torch.cat([tail, qkvb[start: start + n, :channels].float()])  # [taps - 1 + n, channels]
            y = torch.zeros(n, channels)
            for j in range(taps):
                y += x[j: j + n] * conv_w[:, j]
            y = y * torch.sigmoid(y)
            q = y[:, :qk].view(n, kv_heads, dim)
            k = y[:, qk: 2 * qk].view(n, kv_heads, dim)
            q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
            k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
            q_out[start: start + n] = q.reshape(n, qk)
            k_out[start: start + n] = k.reshape(n, qk)
            v_out[start: start + n] = y[:, 2 * qk:]
            state[slot, matrix:] = x[n:].reshape(-1)
        beta.copy_(torch.sigmoid(qkvb[:, channels:].float()))
        rate = torch.exp(A_log)[None, :, None]
        soft = torch.nn.functional.softplus(a.float() + dt_bias).view(-1, heads, dim)
        decay.copy_(torch.exp(-rate * soft).reshape(decay.shape))

    def delta_rule(self, q, k, v, beta, decay, state, slots, ctx, out, heads, kv_heads, dim, vdim):
        rep = heads // kv_heads
        matrix = heads * dim * vdim
        for start, n, slot in zip(ctx.q_starts, ctx.q_lens, slots.tolist()):
            if n == 0:
                continue
            S = state[slot, :matrix].view(heads, vdim, dim).transpose(1, 2).clone()  # [heads, dim, vdim]
            for t in range(start, start + n):
                kt = k[t].view(kv_heads, dim).repeat_interleave(rep, 0)
                qt = q[t].view(kv_heads, dim).repeat_interleave(rep, 0)
                S = decay[t].view(heads, dim)[:, :, None] * S
                u = beta[t][:, None] * (v[t].view(heads, vdim) - torch.einsum("hdv,hd->hv", S, kt))
                S = S + kt[:, :, None] * u[:, None, :]
                out[t] = torch.einsum("hdv,hd->hv", S, qt).reshape(-1)
            state[slot, :matrix] = S.transpose(1, 2).reshape(-1)

    def gated_rms_heads(self, o, weight, eps, gate_pre, out, heads, vdim):
        x = o.view(-1, heads, vdim)
        y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight
        y = y * torch.sigmoid(gate_pre.float().view(-1, heads, vdim))
        out.copy_(y.reshape(out.shape).to(out.dtype))

    # --- routed experts -----------------------------------------------------------------------

    def route_topk(self, x, w_router, groups, keep, ids, weights, bias=None, scoring="softmax", correction=None,
                   group_top=1, weight_scale=1.0):
        n, experts, top = x.shape[0], w_router.shape[0], ids.shape[1]
        logits = x.float() @ w_router.t()
        if scoring == "sigmoid":
            s = torch.sigmoid(logits if bias is None else logits + bias)
            choice = s if correction is None else s + correction
            per = experts // groups
            if keep < groups:
                score = choice.view(n, groups, per).topk(min(group_top, per), dim=-1).values.sum(-1)
                allowed = torch.zeros(n, groups, dtype=torch.bool)
                allowed.scatter_(1, score.topk(keep, dim=-1).indices, True)
                allowed = allowed[:, :, None].expand(-1, -1, per).reshape(n, experts)
                choice = choice.masked_fill(~allowed, float("-inf"))
            chosen = choice.topk(top, dim=-1).indices
            w = s.gather(1, chosen)
            ids.copy_(chosen.to(ids.dtype))
            weights.copy_(w / (w.sum(-1, keepdim=True) + 1e-20) * weight_scale)
            return
        s = (logits if bias is None else logits + bias).softmax(-1)
        per = experts // groups
        best = s.view(n, groups, per).max(-1).values
        allowed = torch.zeros(n, groups, dtype=torch.bool)
        allowed.scatter_(1, best.topk(keep, dim=-1).indices, True)
        allowed = allowed[:, :, None].expand(-1, -1, per).reshape(n, experts)
        chosen = s.masked_fill(~allowed, -1.0).topk(top, dim=-1).indices
        w = s.gather(1, chosen)
        ids.copy_(chosen.to(ids.dtype))
        weights.copy_(w / (w.sum(-1, keepdim=True) + 1e-20) * weight_scale)

    def routed_experts(self, x, ids, weights, w_gate_up, w_down, *, limit, alpha, up_offset, ws, tag="moe"):
        n, top = ids.shape
        out = ws.buffer(tag + ".delta", top * n, w_down.shape[1], torch.float32).view(top, n, -1)
        xf = x.float()
        for t in range(n):
            for j in range(top):
                e = int(ids[t, j])
                g, u = xf[t] @ w_gate_up[e, 0].float().t(), xf[t] @ w_gate_up[e, 1].float().t()
                if limit is not None:
                    g, u = g.clamp(max=limit), u.clamp(-limit, limit)
                y = (g * torch.sigmoid(alpha * g) * (u + up_offset)).to(x.dtype).float()
                out[j, t] = weights[t, j] * (y @ w_down[e].float().t())
        return out

    # --- residual-stream operations of models with norms on both sides of a sublayer ------------

    def bigram_embedding(self, embed, bigram, ids, ctx, state, slots, out, buckets, mul_prev, mul_cur):
        tokens = ids.tolist()
        words = state.view(torch.int32)  # the request's previous token, as the integer's bits
        slot_list = slots.tolist()
        for start, n, first_pos, slot in zip(ctx.q_starts, ctx.q_lens, ctx.start_positions, slot_list):
            if n == 0:
                continue
            for t in range(start, start + n):
                if first_pos + (t - start) == 0:
                    row = buckets
                else:
                    prev = tokens[t - 1] if t > start else int(words[slot, 0])
                    row = (prev * mul_prev + tokens[t] * mul_cur) % buckets
                out[t] = embed[tokens[t]].float() + bigram[row].float()
            words[slot, 0] = tokens[start + n - 1]
        real = sum(ctx.q_lens)
        if real < ids.shape[0]:  # the padding of a fixed-size launch: position 0
            out[real:] = embed[ids[real:].long()].float() + bigram[buckets].float()

    def sandwich_norm(self, h, delta, bias, post_weight, post_eps, weight, eps, out, rows=None, second=None,
                      extra=None):
        x = h if rows is None else h[rows.long()]
        if delta is not None:
            y = delta.sum(0) if delta.dim() == 3 else delta
            if second is not None:
                y = y + (second.sum(0) if second.dim() == 3 else second)
            if extra is not None:
                y = y + extra
            if rows is not None:
                y = y[rows.long()]
            if bias is not None:
                y = y + bias
            if post_weight is not None:
                y = post_weight * (y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + post_eps))
            if rows is None:
                h.add_(y)
                x = h
            else:
                x = x + y
        if out is not None:
            out.copy_((weight * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps))).to(out.dtype))

    def silu_mul_bias(self, gate_up, bias, out):
        i = out.shape[1]
        gu = gate_up.float() + (bias if bias is not None else 0.0)
        g, u = gu[:, :i], gu[:, i:]
        out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))

    def concat_cast(self, a, b, out):
        out.copy_(torch.cat([a, b], dim=-1).to(out.dtype))

    def weighted_sum(self, a, sa, b, sb, out):
        out.copy_(sa * a + sb * b)

    # --- recurrent mixers with a decaying matrix state -------------------------------------------

    def short_conv_residual(self, x, w, state, slots, ctx, out):
        channels, taps = w.shape
        for start, n, slot in zip(ctx.q_starts, ctx.q_lens, slots.tolist()):
            if n == 0:
                continue
            tail = state[slot, : (taps - 1) * channels].view(taps - 1, channels)
            seen = torch.cat([tail, x[start: start + n].float()])  # [taps - 1 + n, channels]
            y = torch.zeros(n, channels)
            for j in range(taps):
                y += seen[j: j + n] * w[:, j]
            out[start: start + n] = (x[start: start + n].float() + y).to(out.dtype)
            if taps > 1:
                state[slot, : (taps - 1) * channels] = seen[n:].reshape(-1)

    def hgrn2_gates(self, proj, bias, lower, write, size):
        q, f = proj[:, :size], proj[:, size: 2 * size]
        q.copy_(q * torch.sigmoid(q))
        f.copy_(lower + (1 - lower) * torch.sigmoid(f + bias))
        write.copy_(1 - f)

    def mlstm_gates(self, gi, gf, bias_i, bias_f, cap, state, m_offset, slots, ctx, gates, heads):
        g = gates.view(-1, heads, 3)
        for start, n, slot in zip(ctx.q_starts, ctx.q_lens, slots.tolist()):
            if n == 0:
                continue
            m = state[slot, m_offset: m_offset + heads].clone()
            for t in range(start, start + n):
                li = cap * torch.tanh((gi[t] + bias_i) / cap)
                lf = torch.nn.functional.logsigmoid(cap * torch.tanh((gf[t] + bias_f) / cap))
                m_new = torch.maximum(lf + m, li)
                g[t, :, 0] = torch.exp(lf + m - m_new)
                g[t, :, 1] = torch.exp(li - m_new)
                g[t, :, 2] = torch.exp(-m_new)
                m = m_new
            state[slot, m_offset: m_offset + heads] = m

    def gated_recurrence(self, q, a, w, gates, v, state, slots, ctx, out, heads, dim, vdim, cols, q_scale):
        matrix = heads * cols * dim
        o = out.view(-1, heads, cols)
        for start, n, slot in zip(ctx.q_starts, ctx.q_lens, slots.tolist()):
            if n == 0:
                continue
            S = state[slot, :matrix].view(heads, cols, dim).transpose(1, 2).clone()  # [heads, dim, cols]
            for t in range(start, start + n):
                qt, wt = q[t].view(heads, dim), w[t].view(heads, dim)
                u = v[t].view(heads, vdim)
                if cols > vdim:
                    u = torch.cat([u, torch.ones(heads, 1)], dim=-1)
                if gates is not None:
                    g = gates[t].view(heads, 3)
                    S = g[:, 0, None, None] * S + wt[:, :, None] * (g[:, 1, None] * u)[:, None, :]
                else:
                    S = a[t].view(heads, dim)[:, :, None] * S + wt[:, :, None] * u[:, None, :]
                o[t] = torch.einsum("hdc,hd->hc", S, qt) * q_scale
            state[slot, :matrix] = S.transpose(1, 2).reshape(-1)

    def lowrank_decay(self, y, w2, bias, tau, decay):
        z = y.float() @ w2.t()
        if bias is not None:
            z = z + bias
        decay.copy_(torch.exp(torch.nn.functional.logsigmoid(z) / tau))

    def recurrence_readout(self, o, gates, weight, eps, gate_pre, out, heads, vdim, cols, gate_act="sigmoid"):
        x = o.view(-1, heads, cols)
        y = x[..., :vdim]
        if gates is not None:
            den = torch.maximum(x[..., vdim].abs(), gates.view(-1, heads, 3)[..., 2]) + 1e-6
            y = y / den[..., None]
        y = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps)
        y = y * (weight.view(heads, vdim) if weight.numel() == heads * vdim else weight)
        if gate_pre is not None:
            g = gate_pre.float().reshape(-1, heads, vdim)
            y = y * (torch.sigmoid(g) if gate_act == "sigmoid" else g * torch.sigmoid(g))
        out.copy_(y.reshape(out.shape).to(out.dtype))

    # --- attention with normalised queries and keys and sigmoid weights ---------------------------

    def qk_norm_rope_write(self, proj, positions, table, rot_dims, q_weight, k_weight, eps, q_out, k_cache,
                           v_cache, slot_mapping, heads, kv_heads, dim, vdim, page_size, bias=None,
                           value_norm=False, values_from_keys=False, interleaved=False):
        n = proj.shape[0]
        end = (heads + kv_heads) * dim + (0 if values_from_keys else kv_heads * vdim)
        proj = proj[:, :end].float()
        if bias is not None:
            proj = proj + bias[:end]
        q = proj[:, : heads * dim].reshape(n, heads, dim)
        k = proj[:, heads * dim: (heads + kv_heads) * dim].reshape(n, kv_heads, dim)
        v = k if values_from_keys else proj[:, (heads + kv_heads) * dim:].reshape(n, kv_heads, vdim)
        if q_weight is not None:
            q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_weight
            k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + eps) * k_weight
        if value_norm:
            v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
        if table is not None and rot_dims > 0:
            half = rot_dims // 2
            cos, sin = table[positions.long(), 0][:, None, :], table[positions.long(), 1][:, None, :]

            def rot(x):
                if interleaved:
                    x1, x2, y = x[..., 0:rot_dims:2], x[..., 1:rot_dims:2], x.clone()
                    y[..., 0:rot_dims:2], y[..., 1:rot_dims:2] = x1 * cos - x2 * sin, x2 * cos + x1 * sin
                    return y
                x1, x2, rest = x[..., :half], x[..., half:rot_dims], x[..., rot_dims:]
                return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin, rest), dim=-1)

            q, k = rot(q), rot(k)
        q_out.copy_(q.reshape(n, heads * dim).to(q_out.dtype))
        if slot_mapping is not None:
            slots = slot_mapping.long()
            page, offset = slots // page_size, slots % page_size
            k_cache[page, :, offset] = k.to(k_cache.dtype)
            v_cache[page, :, offset] = v.to(v_cache.dtype)

    def sigmoid_attention(self, q, k_cache, v_cache, block_tables, ctx, nh, nkv, hd, vdim, page_size, scale,
                          chunk, head_bias, out):
        groups = nh // nkv
        tables = block_tables.long().cpu()
        positions = ctx.positions.cpu().tolist()
        seqs = ctx.seq_of_token.cpu().tolist()
        for t in range(ctx.num_tokens):
            p, s = positions[t], seqs[t]
            lo = (p // chunk) * chunk if chunk else 0
            keys = torch.arange(lo, p + 1)
            pages, offs = tables[s][keys // page_size], keys % page_size
            k = k_cache[pages, :, offs].float().repeat_interleave(groups, dim=1)  # [keys, nh, hd]
            v = v_cache[pages, :, offs].float().repeat_interleave(groups, dim=1)
            scores = torch.einsum("hd,khd->hk", q[t].reshape(nh, hd).float(), k) * scale
            weights = torch.sigmoid(scores + head_bias[:, None])
            out[t] = torch.einsum("hk,khd->hd", weights, v).reshape(nh * vdim).to(out.dtype)

    def sink_attention(self, q, k_cache, v_cache, block_tables, ctx, nh, nkv, hd, vdim, page_size, scale,
                       window, sinks, gate, out, softcap=None, keep_first=0):
        groups = nh // nkv
        tables = block_tables.long().cpu()
        positions = ctx.positions.cpu().tolist()
        seqs = ctx.seq_of_token.cpu().tolist()
        for t in range(ctx.num_tokens):
            p, s = positions[t], seqs[t]
            lo = max(0, p - window + 1) if window else 0
            keys = torch.arange(lo, p + 1)
            if window and keep_first:
                keys = torch.cat([torch.arange(0, min(keep_first, lo)), keys])
            pages, offs = tables[s][keys // page_size], keys % page_size
            k = k_cache[pages, :, offs].float().repeat_interleave(groups, dim=1)  # [keys, nh, hd]
            v = v_cache[pages, :, offs].float().repeat_interleave(groups, dim=1)
            scores = torch.einsum("hd,khd->hk", q[t].reshape(nh, hd).float(), k) * scale
            if softcap:
                scores = softcap * torch.tanh(scores / softcap)
            if sinks is not None:
                scores = torch.cat([scores, sinks[:, None]], dim=1)
            weights = scores.softmax(-1)[:, : keys.numel()]
            o = torch.einsum("hk,khd->hd", weights, v)
            if gate is not None:
                o = o * torch.sigmoid(gate[t].float())[:, None]
            out[t] = o.reshape(nh * vdim).to(out.dtype)

    def gated_add_norm(self, h, delta, gate_pre, gate_bias, weight, eps, out, rows=None):
        if delta.dim() == 3:
            delta = delta.sum(0)
        if gate_pre.dim() == 3:
            gate_pre = gate_pre.sum(0)
        g = gate_pre if gate_bias is None else gate_pre + gate_bias
        if rows is None:
            h.add_(torch.sigmoid(g) * delta)
            x = h
        else:
            r = rows.long()
            x = h[r] + torch.sigmoid(g[r]) * delta[r]
        if out is not None:
            out.copy_((weight * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps))).to(out.dtype))

    def polynorm(self, z, coeff, eps, out):
        x = z.float()
        a, b, c, e = coeff.tolist()

        def unit(y):
            return y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps)

        out.copy_((a * unit(x) + b * unit(x * x) + c * unit(x * x * x) + e).to(out.dtype))

    def linear(self, x, w, out=None, *, ws=None, tag="linear", out_dtype=None, allow_split=False):
        if out is None:
            out = ws.buffer(tag, x.shape[0], w.shape[0], out_dtype)
        out.copy_((x.float() @ w.float().t()).to(out.dtype))
        return out

    def rope_kv_write(self, qkv, positions, table, rotary_dim, q_out, k_cache, v_cache,
                      slot_mapping, nh, nkv, hd, page_size):
        if qkv.dim() == 3:
            qkv = qkv.sum(0)
        n = qkv.shape[0]
        q = qkv[:, : nh * hd].reshape(n, nh, hd).float()
        k = qkv[:, nh * hd: (nh + nkv) * hd].reshape(n, nkv, hd).float()
        v = qkv[:, (nh + nkv) * hd:].reshape(n, nkv, hd).float()
        if table is not None and rotary_dim > 0:
            half = rotary_dim // 2
            cos = table[positions.long(), 0][:, None, :]  # [n, 1, half]
            sin = table[positions.long(), 1][:, None, :]

            def rot(x):
                x1, x2, rest = x[..., :half], x[..., half:rotary_dim], x[..., rotary_dim:]
                return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin, rest), dim=-1)

            q, k = rot(q), rot(k)
        q_out.copy_(q.reshape(n, nh * hd).to(q_out.dtype))
        if slot_mapping is not None:
            slots = slot_mapping.long()
            page, offset = slots // page_size, slots % page_size
            k_cache[page, :, offset] = k.to(k_cache.dtype)
            v_cache[page, :, offset] = v.to(v_cache.dtype)

    def paged_attention(self, q, k_cache, v_cache, block_tables, ctx, nh, nkv, hd, page_size,
                        scale, window, out, ragged=None, value_dim=None):
        vd = hd if value_dim is None else value_dim  # value rows: the first `vd` entries of v_cache's rows
        groups = nh // nkv
        tables = block_tables.long().cpu()
        positions = ctx.positions.cpu().tolist()
        seqs = ctx.seq_of_token.cpu().tolist()
        for t in range(ctx.num_tokens):
            p, s = positions[t], seqs[t]
            lo = max(0, p - window + 1) if window else 0
            keys = torch.arange(lo, p + 1)
            pages = tables[s][keys // page_size].to(k_cache.device)
            offs = (keys % page_size).to(k_cache.device)
            k = k_cache[pages, :, offs].float()  # [keys, nkv, hd]
            v = v_cache[pages, :, offs].float()[..., :vd]
            k = k.repeat_interleave(groups, dim=1)
            v = v.repeat_interleave(groups, dim=1)
            qt = q[t].reshape(nh, hd).float()
            scores = torch.einsum("hd,khd->hk", qt, k) * scale
            probs = scores.softmax(-1)
            out[t] = torch.einsum("hk,khd->hd", probs, v).reshape(nh * vd).to(out.dtype)

    def silu_mul(self, gate_up, out, interleave=0):
        if gate_up.dim() == 3:
            gate_up = gate_up.float().sum(0)
        i = out.shape[1]
        if interleave:  # gates and ups alternate in blocks of `interleave` values
            blocks = gate_up.float().view(gate_up.shape[0], i // interleave, 2, interleave)
            g, u = blocks[:, :, 0].reshape(-1, i), blocks[:, :, 1].reshape(-1, i)
        else:
            g, u = gate_up[:, :i].float(), gate_up[:, i:].float()
        out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))

    def gated_linear(self, x, w_gate_up, interleave, *, ws, tag="ffn", out_dtype=None):
        gate_up = self.linear(x, w_gate_up, ws=ws, tag=tag + ".gate_up", out_dtype=out_dtype or x.dtype)
        act = ws.buffer(tag + ".act", x.shape[0], w_gate_up.shape[0] // 2, out_dtype or x.dtype)
        self.silu_mul(gate_up, act, interleave)
        return act

    def argmax(self, logits, out):
        out.copy_(logits.argmax(-1).to(out.dtype))

    def check_errors(self):
        return None


# --- sampling -----------------------------------------------------------------------------------


def philox_uniforms(seed: int, draw: int, n: int):
    """The uniforms the sampling kernel uses for entries 0..n-1 of a row: Philox4x32-10 with
    counter (i // 4, draw low, draw high, 0) and key (seed low, seed high); entry i takes word
    i % 4; u = ((word >> 9) + 0.5) / 2^23."""
    import numpy as np

    mask = np.uint64(0xFFFFFFFF)
    i = np.arange(n, dtype=np.uint64)
    c0 = i >> np.uint64(2)
    c1 = np.full(n, draw & 0xFFFFFFFF, dtype=np.uint64)
    c2 = np.full(n, (draw >> 32) & 0xFFFFFFFF, dtype=np.uint64)
    c3 = np.zeros(n, dtype=np.uint64)
    k0, k1 = np.uint64(seed & 0xFFFFFFFF), np.uint64((seed >> 32) & 0xFFFFFFFF)
    m0, m1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
    for _ in range(10):
        p0, p1 = m0 * c0, m1 * c2
        hi0, lo0, hi1, lo1 = p0 >> np.uint64(32), p0 & mask, p1 >> np.uint64(32), p1 & mask
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & mask, lo1, (hi0 ^ c3 ^ k1) & mask, lo0
        k0, k1 = (k0 + np.uint64(0x9E3779B9)) & mask, (k1 + np.uint64(0xBB67AE85)) & mask
    words = np.stack([c0, c1, c2, c3], axis=1)[np.arange(n), (i & np.uint64(3)).astype(np.int64)]
    return ((words >> np.uint64(9)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 8388608.0)


def _sample_row(row, temperature, top_k, top_p, min_p, penalty, seen, seed, draw):
    z = row.float().clone()
    if penalty != 1.0 and seen is not None:
        idx = seen.nonzero().flatten()
        z[idx] = torch.where(z[idx] > 0, z[idx] / penalty, z[idx] * penalty)
    if not temperature > 0:
        return int(z.argmax()), None
    z = z * (torch.tensor(1.0) / torch.tensor(temperature, dtype=torch.float32))
    zmax = z.max()
    keep_min = torch.tensor(float("-inf"))
    if 0 < top_k < z.numel():
        keep_min = torch.maximum(keep_min, z.topk(top_k).values[-1])
    if top_p < 1.0:
        kept = z[z >= keep_min].sort(descending=True).values
        mass = torch.exp(kept - zmax)
        target = max(top_p - 1e-6, 0.0) * float(mass.sum())
        first = int((mass.cumsum(0) >= target).nonzero()[0]) if target > 0 else 0
        keep_min = torch.maximum(keep_min, kept[first])
    if min_p > 0.0:
        keep_min = torch.maximum(keep_min, zmax + torch.log(torch.tensor(min_p, dtype=torch.float32)))
    u = torch.from_numpy(philox_uniforms(seed, draw, z.numel()))
    score = z - torch.log(-torch.log(u))
    score[z < keep_min] = float("-inf")
    return int(score.argmax()), score


def _ref_sample(self, logits, out, temperature=None, top_k=None, top_p=None, min_p=None,
                penalty=None, seen_bits=None, seeds=None, draws=None, logprob=None):
    logits_c = logits.float().cpu()
    rows, vocab = logits_c.shape

    def get(t, r, default):
        return default if t is None else t[r].item()

    for r in range(rows):
        seen = None
        if seen_bits is not None:
            words = seen_bits[r].cpu().to(torch.int64) & 0xFFFFFFFF
            seen = ((words[:, None] >> torch.arange(32)[None, :]) & 1).reshape(-1)[:vocab].bool()
        token, _ = _sample_row(logits_c[r], get(temperature, r, 0.0), int(get(top_k, r, 0)),
                               get(top_p, r, 1.0), get(min_p, r, 0.0), get(penalty, r, 1.0), seen,
                               int(get(seeds, r, 0)), int(get(draws, r, 0)))
        out[r] = token
        if logprob is not None:
            logprob[r] = logits_c[r].log_softmax(-1)[token]


RefOps.sample = _ref_sample
