"""A CPU stand-in for the kernel library, for tests only.

The engine has no CPU path.  To check its host logic (batch building, block tables, page
reuse, the run order of layers, the scheduler) on a machine without a GPU, the tests hand
the model this object in place of ``KernelOps``.  It offers the same operations on CPU
tensors with torch arithmetic in float32; it is not bit-exact with the CUDA kernels and is
never imported by the package.
"""
from __future__ import annotations

import math

import torch


class CpuOps:
    def __init__(self, dtype="float32"):
        self.dtype = dtype
        self.act_dtype = torch.float32 if dtype == "float32" else torch.bfloat16
        self.kind = "f32" if dtype == "float32" else "bf16"
        self.launches = 0

    def embed_rows(self, table, tokens, out, scale=1.0):
        out.copy_(table[tokens.long()].float() * scale)

    def rmsnorm_residual(self, d, weight, eps, x, next_weight=None, next_eps=0.0, next_out=None):
        x += (d * torch.rsqrt(d.pow(2).mean(-1, keepdim=True) + eps)) * weight
        if next_out is not None:
            self.rmsnorm(x, next_weight, next_eps, next_out)

    # -- scored attention and the linear recurrence (stand-ins shaped like the kernels' interface) --
    def scored_attention_tile_heights(self, group, dim, vdim):
        return [max(1, 32 // group)]

    def qkv_prepare(self, u, conv_w, conv_state, q_norm, k_norm, eps, cos, sin, ctx, block_table, kcache, vcache, q_out,
                    heads, write_kv_heads, dim, vdim, conv_wt=None, bias=None, vmix_src=None, vmix_lambda=None, v_keep=None):
        n, cols = u.shape
        page = kcache.shape[2]
        if bias is not None:
            u = u + bias
            if conv_state is not None:
                conv_state = conv_state + bias
        y = u.clone()
        if conv_w is not None:
            taps = conv_w.shape[1]
            y.zero_()
            for r in range(n):
                s = int(ctx.row_seq[r])
                row0, pos0, slot = int(ctx.seq_row0[s]), int(ctx.seq_pos0[s]), int(ctx.seq_slot[s])
                for j in range(taps):
                    back = taps - 1 - j
                    if int(ctx.pos[r]) - back < 0:
                        continue
                    src = u[r - back] if r - back >= row0 else conv_state[slot, taps - 1 - (row0 - (r - back))]
                    y[r] += conv_w[:, j] * src
        p = ctx.pos.long()

        def finish(t, size, w):
            t = t.reshape(n, -1, size)
            if w is not None:
                t = t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * w
            if cos is not None:
                pairs = cos.shape[1]
                c, sn = cos[p][:, None, :], sin[p][:, None, :]
                a, b = t[..., 0:2 * pairs:2].clone(), t[..., 1:2 * pairs:2].clone()
                t = t.clone()
                t[..., 0:2 * pairs:2] = a * c - b * sn
                t[..., 1:2 * pairs:2] = b * c + a * sn
            return t

        q_out.copy_(finish(y[:, :heads * dim], dim, q_norm).reshape(n, -1).to(q_out.dtype))
        if not write_kv_heads:
            return
        g = write_kv_heads
        k = finish(y[:, heads * dim:(heads + g) * dim], dim, k_norm)
        v = y[:, (heads + g) * dim:].reshape(n, g, vdim) if vcache is not None else None
        if vmix_src is not None:
            lam = float(vmix_lambda[0])
            v = (1.0 - lam) * v + lam * vmix_src.reshape(n, g, vdim)
        if v_keep is not None:
            v_keep.copy_(v.reshape(n, -1))
        for r in range(n):
            blk = int(block_table[int(ctx.row_seq[r]), int(p[r]) // page])
            kcache[blk, :, int(p[r]) % page, :] = k[r].to(kcache.dtype)
            if v is not None:
                vcache[blk, :, int(p[r]) % page, :] = v[r].to(vcache.dtype)

    def conv_state_update(self, u, state, ctx, taps, tiles):
        t_seq, t_row0, t_rows, count = tiles
        for i in range(count):
            s, row0, cnt = int(t_seq[i]), int(t_row0[i]), int(t_rows[i])
            slot, pos0 = int(ctx.seq_slot[s]), int(ctx.seq_pos0[s])
            old = state[slot].clone()
            for j in range(taps - 1):
                pos = pos0 + cnt - (taps - 1) + j
                if pos < 0:
                    state[slot, j] = 0
                elif pos >= pos0:
                    state[slot, j] = u[row0 + pos - pos0]
                else:
                    state[slot, j] = old[pos - pos0 + taps - 1]

    def scored_attention(self, q, kcache, vcache, block_table, out, heads, kv_heads, dim, vdim, scale, softcap, sink,
                         slopes, window, ctx, dist_a=None, dist_b=None, sinks=None, keep_first=0):
        n = q.shape[0]
        page = kcache.shape[2]
        grp = heads // kv_heads
        for r in range(n):
            p = int(ctx.pos[r])
            lo = max(0, p - window + 1) if window else 0
            idx = torch.arange(lo, p + 1)
            if window and keep_first and lo > 0:
                idx = torch.cat([torch.arange(0, min(keep_first, lo)), idx])
            blocks = block_table[int(ctx.row_seq[r])][(idx // page).long()].long()
            slots = (idx % page).long()
            k = kcache[blocks, :, slots, :].float().repeat_interleave(grp, dim=1)
            v = k if vcache is None else vcache[blocks, :, slots, :].float().repeat_interleave(grp, dim=1)
            s = torch.einsum("hd,khd->hk", q[r].float().view(heads, dim), k) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            if slopes is not None:
                s = s - slopes[:, None] * (p - idx).float()[None, :]
            if dist_a is not None:
                s = s - dist_a[:, None] * torch.log1p(dist_b[:, None] * (p - idx).float()[None, :])
            m = s.max(-1, keepdim=True).values
            e = torch.exp(s - m)
            extra = torch.exp((sinks[:, None] if sinks is not None else 0.0) - m) if sink else 0.0
            den = e.sum(-1, keepdim=True) + extra
            out[r] = torch.einsum("hk,khd->hd", e / den, v).reshape(-1).to(out.dtype)

    # -- kernels on the stream, the second embedding table and the routed feed-forward (stand-ins) --
    def embed_pair(self, table, pair_table, ctx, last_token, out, scale, buckets, mul_prev, mul_cur):
        for r in range(out.shape[0]):
            s, tok = int(ctx.row_seq[r]), int(ctx.tokens[r])
            row = buckets
            if int(ctx.pos[r]) > 0:
                prev = int(ctx.tokens[r - 1]) if r > int(ctx.seq_row0[s]) else int(last_token[int(ctx.seq_slot[s])])
                row = (prev * mul_prev + tok * mul_cur) % buckets
            out[r] = table[tok].float() * scale + pair_table[row].float()

    def last_token_update(self, ctx, last_token, tiles):
        t_seq, t_row0, t_rows, count = tiles
        for i in range(count):
            last_token[int(ctx.seq_slot[int(t_seq[i])])] = int(ctx.tokens[int(t_row0[i]) + int(t_rows[i]) - 1])

    def norm_conv(self, x, weight, eps, taps_t, state, state_col0, ctx, out, normed, normed_col0):
        n, width = out.shape
        taps = taps_t.shape[0]
        h = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight
        normed[:, normed_col0:normed_col0 + width] = h
        for r in range(n):
            s = int(ctx.row_seq[r])
            row0, slot = int(ctx.seq_row0[s]), int(ctx.seq_slot[s])
            acc = torch.zeros(width)
            for j in range(taps):
                back = taps - 1 - j
                if int(ctx.pos[r]) - back < 0:
                    continue
                src = h[r - back] if r - back >= row0 else state[slot, taps - 1 - (row0 - (r - back)), state_col0:state_col0 + width]
                acc += taps_t[j] * src
            out[r] = (h[r] + acc).to(out.dtype)

    def scaled_add(self, x, scale, d, rounded=None):
        if scale is not None:
            x += scale * d
        if rounded is not None:
            rounded.copy_(x.to(rounded.dtype))

    def token_gate(self, t, table, col0, tokens, out):
        e = table[tokens.long()][:, col0:col0 + t.shape[1]].float()
        out.copy_((torch.nn.functional.gelu(t, approximate="tanh") * e).to(out.dtype))

    def normed_add_mix(self, x, y, weight, eps, mult, history, index, mix):
        if y is not None:
            x += mult * (y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps) * weight)
        if history is not None:
            width = x.shape[1]
            history[:, index * width:(index + 1) * width] = x
            x.copy_(sum(mix[j] * history[:, j * width:(j + 1) * width] for j in range(index + 1)))

    def copy_history(self, x, history):
        history[:, :x.shape[1]] = x

    def glu_clamped(self, gate_up, out, limit, alpha):
        inter = out.shape[1]
        g = gate_up[:, :inter].float().clamp(max=limit)
        u = gate_up[:, inter:].float().clamp(-limit, limit)
        out.copy_((g * torch.sigmoid(alpha * g) * (u + 1.0)).to(out.dtype))

    def route(self, logits, correction, groups, keep, top, weight_scale, chosen, weights, softmax_top=False):
        if groups != 1 or not softmax_top:
            raise NotImplementedError("the stand-in routes by the largest logits only")
        z = logits if correction is None else logits + correction
        order = torch.sort(z, dim=-1, descending=True, stable=True).indices[:, :top]
        chosen.copy_(order.to(torch.int32))
        weights.copy_(torch.softmax(torch.gather(logits, 1, order), -1) * weight_scale)

    def group_rows(self, chosen, experts, group_off, tile_prefix, order, place):
        pairs = chosen.numel()
        self._entry_expert = chosen.reshape(-1).long().clone()
        order.reshape(-1)[:pairs] = torch.arange(pairs, dtype=torch.int32)
        place.reshape(-1)[:pairs] = torch.arange(pairs, dtype=torch.int32)

    def grouped_linear(self, x, w, out, rows, x_group_cols=0, o_group_cols=0, lists=None, order_div=1, gather=True,
                       sorted_x=None):
        if lists is None:
            # one product per group over the same rows: group g reads the columns g * x_group_cols .. + k of x
            # and writes the columns g * o_group_cols .. + n of out (w: [groups, n, k])
            groups, n_out, k = w.shape
            for g in range(groups):
                src = x[:rows, g * x_group_cols:g * x_group_cols + k].float()
                out[:rows, g * o_group_cols:g * o_group_cols + n_out] = (src @ w[g].float().t()).to(out.dtype)
            return
        order = lists[2].reshape(-1)
        for i in range(rows):
            src = x[int(order[i]) // order_div] if gather else x[i]
            out[i] = (w[int(self._entry_expert[i])].float() @ src.float()).to(out.dtype)

    def combine(self, x, d, y, place, weights, top, scale=None):
        n = x.shape[0]
        add = (weights[:, :, None] * y[place.reshape(-1).long()[:n * top]].view(n, top, -1)).sum(1)
        if d is not None:
            add = add + d
        x += add if scale is None else scale * add

    def gla_scan(self, u, z, bias, tau, state, norm_w, eps, out, heads, dim, vdim, q_scale, ctx, tiles, scratch=None):
        t_seq, t_row0, t_rows, count = tiles
        hd, hv = heads * dim, heads * vdim
        for i in range(count):
            s, row0, cnt = int(t_seq[i]), int(t_row0[i]), int(t_rows[i])
            slot = int(ctx.seq_slot[s])
            S = state[slot]
            if int(ctx.seq_pos0[s]) == 0:
                S.zero_()
            for r in range(row0, row0 + cnt):
                qv = u[r, :hd].view(heads, dim) * q_scale
                kv = u[r, hd:2 * hd].view(heads, dim)
                vv = u[r, 2 * hd:2 * hd + hv].view(heads, vdim)
                gate = u[r, 2 * hd + hv:]
                decay = torch.exp(torch.nn.functional.logsigmoid(z[r] + bias) / tau).view(heads, dim)
                S.mul_(decay[:, :, None]).add_(kv[:, :, None] * vv[:, None, :])
                o = torch.einsum("hd,hde->he", qv, S)
                o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps) * norm_w
                out[r] = (o.reshape(-1) * gate * torch.sigmoid(gate)).to(out.dtype)

    def rmsnorm(self, x, weight, eps, out, rows=None):
        src = x if rows is None else x[rows.long()]
        inv = torch.rsqrt(src.pow(2).mean(-1, keepdim=True) + eps)
        out.copy_(((src * inv) * weight).to(out.dtype))

    def linear(self, x, w, out, residual=None):
        y = x.float() @ w.float().t()
        if residual is not None:
            y = residual + y
        out.copy_(y.to(out.dtype))

    def fuses_swiglu(self, width, intermediate, activation="silu"):
        return False

    # -- layer norm, latent attention and the element-wise steps of gated designs ---------------------
    @staticmethod
    def _layer_normed(t, eps):
        c = t - t.mean(-1, keepdim=True)
        return c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + eps)

    def layernorm(self, x, weight, eps, out, rows=None, weight2=None, out2=None):
        src = x if rows is None else x[rows.long()]
        n = self._layer_normed(src.float(), eps)
        out.copy_((n * weight).to(out.dtype))
        if out2 is not None:
            out2.copy_((n * weight2).to(out2.dtype))

    def layernorm_residual(self, d, weight, eps, x, next_weight=None, next_eps=0.0, next_out=None):
        x += self._layer_normed(d, eps) * weight
        if next_out is not None:
            self.layernorm(x, next_weight, next_eps, next_out)

    @staticmethod
    def _turn(t, p, cos, sin, half_layout):
        """t: [n, ..., size]; the first 2 * pairs entries turn by the tables' rows p."""
        if cos is None:
            return t
        pairs = cos.shape[1]
        shape = (t.shape[0],) + (1,) * (t.dim() - 2) + (pairs,)
        c, s = cos[p].reshape(shape), sin[p].reshape(shape)
        out = t.clone()
        if half_layout:
            a, b = t[..., :pairs], t[..., pairs:2 * pairs]
            out[..., :pairs], out[..., pairs:2 * pairs] = a * c - b * s, b * c + a * s
        else:
            a, b = t[..., 0:2 * pairs:2], t[..., 1:2 * pairs:2]
            out[..., 0:2 * pairs:2], out[..., 1:2 * pairs:2] = a * c - b * s, b * c + a * s
        return out

    def latent_store(self, d, weight, eps, pos, row_seq, cos, sin, block_table, cache, rank, rot_dim, half_layout=False,
                     q_latent=None):
        page = cache.shape[1]
        if q_latent is not None:
            q_w, q_out = q_latent
            cq = d[:, rank + rot_dim:rank + rot_dim + q_w.shape[0]]
            q_out.copy_((cq * torch.rsqrt(cq.pow(2).mean(-1, keepdim=True) + eps) * q_w).to(q_out.dtype))
        p = pos.long()
        c = d[:, :rank]
        c = c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + eps) * weight
        kr = self._turn(d[:, rank:rank + rot_dim], p, cos, sin, half_layout)
        for r in range(d.shape[0]):
            blk = int(block_table[int(row_seq[r]), int(p[r]) // page])
            cache[blk, int(p[r]) % page] = torch.cat([c[r], kr[r]]).to(cache.dtype)

    def rotate_heads(self, q, heads, head_stride, offset, rot_dim, out, out_head_stride, out_offset, pos, cos, sin,
                     half_layout=False):
        n = q.shape[0]
        src = q.float().reshape(n, -1)[:, :heads * head_stride].reshape(n, heads, head_stride)[..., offset:offset + rot_dim]
        turned = self._turn(src, pos.long(), cos, sin, half_layout)
        dst = out.reshape(n, -1)[:, :heads * out_head_stride].reshape(n, heads, out_head_stride)
        dst[..., out_offset:out_offset + rot_dim] = turned.to(out.dtype)

    def latent_attention_tile_heights(self, heads, rank, rot_dim):
        return [max(1, 32 // heads)]

    def latent_attention(self, q, cache, block_table, out, heads, rank, rot_dim, scale, ctx, window=0, sinks=None):
        page = cache.shape[1]
        dk = rank + rot_dim
        for r in range(q.shape[0]):
            p = int(ctx.pos[r])
            idx = torch.arange(max(0, p - window + 1) if window else 0, p + 1)
            keys = cache[block_table[int(ctx.row_seq[r])][(idx // page).long()].long(), (idx % page).long()].float()
            s = (q[r].float().view(heads, dk) @ keys.t()) * scale
            m = s.max(-1, keepdim=True).values
            if sinks is not None:
                m = torch.maximum(m, sinks.view(-1, 1))
            e = torch.exp(s - m)
            den = e.sum(-1, keepdim=True) + (torch.exp(sinks.view(-1, 1) - m) if sinks is not None else 0.0)
            out[r] = ((e / den) @ keys[:, :rank]).reshape(-1).to(out.dtype)

    def sigmoid_gate(self, v, g, group=1):
        v.copy_((v.float() * torch.sigmoid(g.float()).repeat_interleave(group, dim=1)).to(v.dtype))

    def glu_gelu(self, gate_up, out):
        inter = out.shape[1]
        g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
        gelu = 0.5 * g * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (g + 0.044715 * g ** 3)))
        out.copy_((gelu * u).to(out.dtype))

    def softcap_rows(self, z, cap):
        z.copy_(cap * torch.tanh(z / cap))

    def rope_cache(self, qkv, pos, row_seq, cos, sin, block_table, kcache, vcache, heads, kv_heads, head_dim,
                   write_kv=True):
        n = qkv.shape[0]
        page = kcache.shape[2]
        half = head_dim // 2
        q = qkv[:, :heads * head_dim].view(n, heads, head_dim).float()
        k = qkv[:, heads * head_dim:(heads + kv_heads) * head_dim].view(n, kv_heads, head_dim).float()
        v = qkv[:, (heads + kv_heads) * head_dim:].view(n, kv_heads, head_dim)
        if cos is not None:
            c = cos[pos.long()][:, None, :]
            s = sin[pos.long()][:, None, :]

            def rot(t):
                x1, x2 = t[..., :half], t[..., half:]
                return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)

            q, k = rot(q), rot(k)
        qkv[:, :heads * head_dim] = q.reshape(n, -1).to(qkv.dtype)
        if not write_kv:
            return
        for r in range(n):
            p = int(pos[r])
            blk = int(block_table[int(row_seq[r]), p // page])
            kcache[blk, :, p % page, :] = k[r].to(kcache.dtype)
            vcache[blk, :, p % page, :] = v[r]

    def attention(self, qkv, kcache, vcache, block_table, row_seq, pos, out, heads, kv_heads, head_dim, window,
                  max_keys, scale, batch=None):
        n = qkv.shape[0]
        page = kcache.shape[2]
        grp = heads // kv_heads
        for r in range(n):
            p = int(pos[r])
            lo = max(0, p - window + 1) if window and window > 0 else 0
            table = block_table[int(row_seq[r])]
            idx = torch.arange(lo, p + 1)
            blocks = table[(idx // page).long()].long()
            slots = (idx % page).long()
            k = kcache[blocks, :, slots, :].float()  # [keys, kv_heads, hd]
            v = vcache[blocks, :, slots, :].float()
            q = qkv[r, :heads * head_dim].view(heads, head_dim).float()
            kk = k.repeat_interleave(grp, dim=1)
            vv = v.repeat_interleave(grp, dim=1)
            s = torch.einsum("hd,khd->hk", q, kk) * scale
            w = torch.softmax(s, dim=-1)
            out[r] = torch.einsum("hk,khd->hd", w, vv).reshape(-1).to(out.dtype)

    def swiglu(self, gate_up, out):
        inter = out.shape[1]
        g = gate_up[:, :inter].float()
        u = gate_up[:, inter:].float()
        out.copy_((g * torch.sigmoid(g) * u).to(out.dtype))

    def sample_rows(self, logits, temperature, uniform, out_tokens):
        for r in range(logits.shape[0]):
            t = float(temperature[r])
            row = logits[r]
            if t <= 0:
                out_tokens[r] = int(torch.argmax(row))  # torch returns the first maximum on CPU
                mx = row.max()
                out_tokens[r] = int((row == mx).nonzero()[0])
            else:
                w = torch.exp((row - row.max()) / t).double()
                cum = torch.cumsum(w, 0)
                target = float(uniform[r]) * float(cum[-1])
                hit = (cum > target).nonzero()
                out_tokens[r] = int(hit[0]) if len(hit) else int((w > 0).nonzero()[-1])

    def fingerprint_rows(self, logits, slot, state):
        import struct
        mask = (1 << 64) - 1

        def mix64(z):
            z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
            z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
            return z ^ (z >> 31)

        for r in range(logits.shape[0]):
            s = int(slot[r])
            h = int(state[s]) & mask
            data = logits[r].contiguous().numpy().tobytes()
            i = 0
            while i + 8 <= len(data):
                (wd,) = struct.unpack_from("<Q", data, i)
                h = ((h ^ wd) * 1099511628211) & mask
                i += 8
            while i < len(data):
                h = ((h ^ data[i]) * 1099511628211) & mask
                i += 1
            h = mix64(h)
            state[s] = h - (1 << 64) if h >= (1 << 63) else h
