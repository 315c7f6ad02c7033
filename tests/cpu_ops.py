"""A test double of the kernel interface (llmengine.ops.CudaOps) in plain PyTorch on the CPU.

It exists so that the host-side logic of the engine (batch building, block tables, page reuse,
scheduling, the wiring of parts) can be exercised where there is no GPU. It is never imported by
the package; the product path runs only on the CUDA kernels. Semantics follow the docstrings of
llmengine/ops.py, not the kernels' code.
"""
from __future__ import annotations


import numpy as np
import torch


class CpuOps:
    def embed(self, table, ids, out, scale=1.0):
        n = out.shape[0]
        out.copy_(table[ids[:n].long()].float() * scale)
        return out

    def rmsnorm(self, h, weight, eps, out, delta=None, rows=None, n_rows=None, write_back=True, center=False):
        if rows is not None:
            n = rows.numel() if n_rows is None else n_rows
            idx = rows[:n].long()
            x = h[idx].clone()
            if delta is not None:
                d = delta if delta.dim() == 2 else delta.sum(0)
                x = x + d[idx]
        else:
            n = h.shape[0] if n_rows is None else n_rows
            x = h[:n]
            if delta is not None:
                d = delta if delta.dim() == 2 else delta.sum(0)
                x = x + d[:n]
                if write_back:
                    h[:n] = x
        if center:
            x = x - x.mean(-1, keepdim=True)
        ss = (x * x).sum(-1, keepdim=True)
        inv = 1.0 / torch.sqrt(ss / x.shape[-1] + eps)
        out[:n] = ((weight * x) * inv).to(out.dtype)
        return out

    def softcap(self, x, cap):
        x.copy_(cap * torch.tanh(x / cap))
        return x

    def residual_add(self, h, delta, n_rows=None):
        n = h.shape[0] if n_rows is None else n_rows
        d = delta if delta.dim() == 2 else delta.sum(0)
        h[:n] += d[:n]
        return h

    @staticmethod
    def _glu(g, u, act):
        if isinstance(act, tuple):  # ("clamped_swish", limit, slope)
            _, lim, slope = act
            g, u = torch.clamp(g, max=lim), torch.clamp(u, -lim, lim)
            return g * torch.sigmoid(slope * g) * (u + 1.0)
        return CpuOps._act(g, act) * u

    @staticmethod
    def _act(g, act):
        if act == "gelu_tanh":
            return 0.5 * g * (1.0 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))
        return g / (1.0 + torch.exp(-g))

    def silu_mul(self, gate_up, out, block=0, act="silu"):
        ff = out.shape[1]
        if block:
            gu = gate_up.float().view(gate_up.shape[0], ff // block, 2, block)
            g, u = gu[:, :, 0].reshape(-1, ff), gu[:, :, 1].reshape(-1, ff)
        else:
            g = gate_up[:, :ff].float()
            u = gate_up[:, ff:].float()
        out.copy_(self._glu(g, u, act).to(out.dtype))
        return out

    def gemm(self, a, w, out, ws=None):
        out.copy_((a.float() @ w.float().t()).to(out.dtype))
        return out

    def gemm_partials(self, a, w, ws, tag):
        parts = ws.get(tag, (2, a.shape[0], w.shape[0]), torch.float32)  # two parts, to exercise the consumers
        half = a.shape[1] // 2
        parts[0] = a[:, :half].float() @ w[:, :half].float().t()
        parts[1] = a[:, half:].float() @ w[:, half:].float().t()
        return parts

    def reduce_partials(self, parts, out):
        out.copy_(parts.sum(0).to(out.dtype))
        return out

    def silu_mul_partials(self, parts, out, block=0, act="silu"):
        return self.silu_mul(parts.sum(0), out, block, act)

    def gemm_swiglu(self, a, w_blocked, out, ws=None, act="silu"):
        gate_up = (a.float() @ w_blocked.float().t())
        return self.silu_mul(gate_up, out, 128, act)

    # ------------------------------------------------------------------ stream, token side input
    def stream_add(self, h, a, b=None, copy=None, n_rows=None):
        n = h.shape[0] if n_rows is None else n_rows
        for d in (a, b):
            if d is not None:
                h[:n] += (d if d.dim() == 2 else d.sum(0))[:n]
        if copy is not None:
            copy[:n] = h[:n].to(copy.dtype)
        return h

    def token_gate(self, z, table, col0, ids, out):
        n, dim = out.shape
        e = table[ids[:n].long(), col0:col0 + dim].float()
        out.copy_((self._act(z.float(), "gelu_tanh") * e).to(out.dtype))
        return out

    # ------------------------------------------------------------------ latent attention
    def latent_prep(self, parts, q_off, q_rank, kv_off, kv_rank, rot_dim, rot_dims, wq, wkv, eps, cos, sin, batch, block_table, cq, cache):
        n = batch.n_tokens
        x = parts.sum(0)[:n]
        q = x[:, q_off:q_off + q_rank]
        cq[:n] = (q / torch.sqrt((q * q).mean(-1, keepdim=True) + eps) * wq).to(cq.dtype)
        if cache is None:
            return
        c = x[:, kv_off:kv_off + kv_rank]
        c = c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * wkv
        kr = x[:, kv_off + kv_rank:kv_off + kv_rank + rot_dim].clone()
        half, ps = rot_dims // 2, cache.shape[2]
        for t in range(n):
            pos = int(batch.positions[t])
            if half:
                u, v = kr[t, :half].clone(), kr[t, half:rot_dims].clone()
                kr[t, :half] = u * cos[pos] - v * sin[pos]
                kr[t, half:rot_dims] = v * cos[pos] + u * sin[pos]
            page = int(block_table[int(batch.token_seq[t]), pos // ps])
            assert page >= 0, "write into a page that was given back"
            cache[page, 0, pos % ps] = torch.cat([c[t], kr[t]]).to(cache.dtype)

    def heads_product(self, a, w, out, gate=None, gate_off=0):
        y = torch.einsum("thk,hnk->thn", a.float(), w.float())
        if gate is not None:
            n, H, N = out.shape
            g = gate.sum(0)[:n, gate_off:gate_off + H * N].view(n, H, N)
            y = y * torch.sigmoid(g)
        out.copy_(y.to(out.dtype))
        return out

    def latent_query(self, q, wkt, ql, heads, dim, rot_dim, kv_rank, rot_dims, cos, sin, positions, absorb=True):
        n = ql.shape[0]
        qh = q[:n].float().view(n, heads, dim + rot_dim)
        if absorb:
            ql[:, :, :kv_rank] = torch.einsum("thd,hrd->thr", qh[:, :, :dim], wkt.float()).to(ql.dtype)
        r = qh[:, :, dim:].clone()
        half = rot_dims // 2
        if half:
            pos = positions[:n].long()
            c, s = cos[pos][:, None, :], sin[pos][:, None, :]
            u, v = r[:, :, :half].clone(), r[:, :, half:rot_dims].clone()
            r[:, :, :half] = u * c - v * s
            r[:, :, half:rot_dims] = v * c + u * s
        ql[:, :, kv_rank:] = r.to(ql.dtype)
        return ql

    def latent_attention(self, ql, cache, batch, block_table, out, kv_rank, scale, window=0):
        ps = cache.shape[2]
        for t in range(batch.n_tokens):
            pos = int(batch.positions[t])
            lo = max(0, pos - window + 1) if window > 0 else 0
            idx = torch.arange(lo, pos + 1)
            pages = block_table[int(batch.token_seq[t])][(idx // ps).long()].long()
            assert (pages >= 0).all(), "read from a page that was given back"
            rows = cache[pages, 0, (idx % ps).long(), :].float()  # [S, Dk]
            p = torch.softmax((ql[t].float() @ rows.t()) * scale, dim=-1)  # [H, S]
            out[t] = (p @ rows[:, :kv_rank]).to(out.dtype)
        return out

    def sigmoid_gate(self, x, gate, gate_off):
        n, cols = x.shape
        x.copy_((x.float() * torch.sigmoid(gate.sum(0)[:n, gate_off:gate_off + cols])).to(x.dtype))
        return x

    # ------------------------------------------------------------------ routed feed-forward
    def route(self, x, w, bias, top, idx, share):
        z = x.float() @ w.float().t()
        if bias is not None:
            z = z + bias
        order = torch.argsort(z, dim=-1, descending=True, stable=True)[:, :top]
        idx.copy_(order.to(torch.int32))
        share.copy_(torch.softmax(torch.gather(z, 1, order), dim=-1))

    def route_grouped(self, x, w, correction, top, groups, keep, norm_eps, idx, share, score="softmax", group_top=1, normalize=True,
                      weight_scale=1.0, gate_out=None):
        z = x.float() @ w.float().t()
        if gate_out is not None:  # one more row behind the router's: a gate's logit
            gate_out[:z.shape[0]] = torch.sigmoid(z[:, -1])
            z = z[:, :-1]
        s = torch.sigmoid(z) if score == "sigmoid" else torch.softmax(z, dim=-1)
        choice = s + correction if correction is not None else s.clone()
        E = s.shape[1]
        per = E // groups
        if keep < groups:
            best = torch.sort(choice.view(-1, groups, per), dim=-1, descending=True).values[..., :min(group_top, per)].sum(-1)
            kept = torch.argsort(best, dim=-1, descending=True, stable=True)[:, :keep]
            mask = torch.zeros(s.shape[0], groups, dtype=torch.bool)
            mask.scatter_(1, kept, True)
            choice = torch.where(mask.repeat_interleave(per, dim=1), choice, torch.full_like(choice, float("-inf")))
        order = torch.argsort(choice, dim=-1, descending=True, stable=True)[:, :top]
        picked = torch.gather(s, 1, order)
        idx.copy_(order.to(torch.int32))
        share.copy_((picked / (picked.sum(-1, keepdim=True) + norm_eps) if normalize else picked) * weight_scale)

    def routed_tile_rows(self, n_tokens=0, dtype=None, inner=(), per_expert=0.0):
        return 4

    def routed_group(self, idx, experts, tile, ws, tag, real_experts=None):
        flat = idx.reshape(-1).tolist()
        tiles_e, tiles_r = [], []
        for e in range(experts if real_experts is None else real_experts):
            rows = [p for p, ex in enumerate(flat) if ex == e]
            for i in range(0, len(rows), tile):
                chunk = rows[i:i + tile]
                tiles_e.append(e)
                tiles_r.append(chunk + [-1] * (tile - len(chunk)))
        cap = (len(flat) + tile - 1) // tile + experts
        while len(tiles_e) < cap:
            tiles_e.append(-1)
            tiles_r.append([-1] * tile)
        return torch.tensor(tiles_e, dtype=torch.int32), torch.tensor(tiles_r, dtype=torch.int32)

    def routed_product(self, a, a_div, w, tile_expert, tile_rows, out, epilogue, share=None, act="silu"):
        for e, rows in zip(tile_expert.tolist(), tile_rows.tolist()):
            if e < 0:
                continue
            for p in rows:
                if p < 0:
                    continue
                v = w[e].float() @ a[p // a_div].float()
                if epilogue == "gelu":
                    v = 0.5 * v * (1.0 + torch.erf(v / 2.0 ** 0.5))
                elif epilogue == "share":
                    v = v * share[p]
                elif epilogue == "gated_pairs":
                    v = self._glu(v[0::2], v[1::2], act)
                else:  # "silu_pairs": rows 2 f and 2 f + 1 are a gate and its up row
                    v = torch.nn.functional.silu(v[0::2]) * v[1::2]
                out[p] = v.to(out.dtype)
        return out

    def routed_combine(self, y, out, top, identity=None, extra=None, extra_gate=None):
        n = out.shape[0]
        rows = y.view(n, top, -1).clone()
        if identity is not None:
            idx, share, real, x = identity
            own = (idx >= real)[:, :, None]
            rows = torch.where(own, share[:, :, None] * x[:n].float()[:, None, :], rows)
        total = rows.sum(1)
        if extra is not None:
            b = (extra if extra.dim() == 2 else extra.sum(0))[:n]
            total = total + (b * extra_gate[:n, None] if extra_gate is not None else b)
        out.copy_(total)
        return out

    def rope_kv_write(self, qkv, positions, token_seq, block_table, cos, sin, kcache, vcache, n_tokens, nq, nkv, hd, parts=None):
        half = hd // 2
        src = qkv if parts is None else parts.sum(0)
        for t in range(n_tokens):
            pos = int(positions[t])
            row = src[t].float()
            q = row[: nq * hd].view(nq, hd).clone()
            k = row[nq * hd:(nq + nkv) * hd].view(nkv, hd).clone()
            v = row[(nq + nkv) * hd:].view(nkv, hd)
            if cos is not None:
                c, s = cos[pos], sin[pos]
                for x in (q, k):
                    a, b = x[:, :half].clone(), x[:, half:].clone()
                    x[:, :half] = a * c - b * s
                    x[:, half:] = b * c + a * s
            qkv[t, : nq * hd] = q.reshape(-1).to(qkv.dtype)
            if kcache is not None:
                ps = kcache.shape[2]
                page = int(block_table[int(token_seq[t]), pos // ps])
                assert page >= 0, "write into a page that was given back"
                kcache[page, :, pos % ps, :] = k.to(kcache.dtype)
                vcache[page, :, pos % ps, :] = v.to(vcache.dtype)
            else:
                qkv[t, nq * hd:(nq + nkv) * hd] = k.reshape(-1).to(qkv.dtype)

    # ------------------------------------------------------------------ norms on the outputs, gated attention, selective scan
    def norm_add(self, h, a, b, weight, layer_scale, eps, copy=None, n_rows=None):
        n = h.shape[0] if n_rows is None else n_rows
        y = (a if a.dim() == 2 else a.sum(0))[:n].clone()
        if b is not None:
            y = y + (b if b.dim() == 2 else b.sum(0))[:n]
        v = y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * weight
        h[:n] += v * layer_scale if layer_scale is not None else v
        if copy is not None:
            copy[:n] = h[:n].to(copy.dtype)
        return h

    def qkv_prep(self, parts, heads, kv_heads, dk, dv, q_norm, k_norm, eps, cos, sin, batch, block_table, q_out, kcache, vcache,
                 mix_role=0, mix_weight=None, v_first=None, norm_wide=False):
        src = parts.sum(0)
        half = 0 if cos is None else cos.shape[1]
        for t in range(batch.n_tokens):
            pos = int(batch.positions[t])
            row = src[t].float()
            q = row[:heads * dk].view(heads, dk).clone()
            k = row[heads * dk:(heads + kv_heads) * dk].view(kv_heads, dk).clone()
            v = row[(heads + kv_heads) * dk:(heads + kv_heads) * dk + kv_heads * dv].clone()
            for x, w in ((q, q_norm), (k, k_norm)):
                if w is not None and x.numel() and norm_wide:  # one norm over the whole projection, a weight a number
                    x.copy_(x / torch.sqrt((x * x).mean() + eps) * w.view(x.shape))
                elif w is not None and x.numel():
                    x.copy_(x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w)
                if half:
                    a, b = x[:, :half].clone(), x[:, half:2 * half].clone()
                    x[:, :half] = a * cos[pos] - b * sin[pos]
                    x[:, half:2 * half] = b * cos[pos] + a * sin[pos]
            if mix_role == 1:
                v_first[t] = v
            elif mix_role == 2:
                v = (1.0 - mix_weight) * v + mix_weight * v_first[t]
            q_out[t] = q.reshape(-1).to(q_out.dtype)
            if kcache is not None:
                ps = kcache.shape[2]
                page = int(block_table[int(batch.token_seq[t]), pos // ps])
                assert page >= 0, "write into a page that was given back"
                kcache[page, :, pos % ps, :] = k.to(kcache.dtype)
                vcache[page, :, pos % ps, :] = v.view(kv_heads, dv).to(vcache.dtype)

    def gated_attention(self, q, kcache, vcache, batch, block_table, out, nq, nkv, dk, dv, scale, window=0, chunk=0, sink=None,
                        gate=None, gate_off=0, gate_per_head=False):
        ps, g = kcache.shape[2], nq // nkv
        gates = gate.sum(0) if gate is not None else None
        for t in range(batch.n_tokens):
            pos = int(batch.positions[t])
            lo = max(0, pos - window + 1) if window > 0 else 0
            if chunk > 0:
                lo = max(lo, (pos // chunk) * chunk)
            idx = torch.arange(lo, pos + 1)
            pages = block_table[int(batch.token_seq[t])][(idx // ps).long()].long()
            assert (pages >= 0).all(), "read from a page that was given back"
            K = kcache[pages, :, (idx % ps).long(), :].float()
            V = vcache[pages, :, (idx % ps).long(), :].float()
            qt = q[t].float().view(nq, dk)
            for h in range(nq):
                s = (K[:, h // g, :] @ qt[h]) * scale
                if sink is not None:
                    p = torch.softmax(torch.cat([s, sink[h:h + 1]]), dim=0)[:-1]
                else:
                    p = torch.softmax(s, dim=0)
                o = p @ V[:, h // g, :]
                if gates is not None and gate_per_head:
                    o = o * torch.sigmoid(gates[t, gate_off + h])
                elif gates is not None:
                    o = o * torch.sigmoid(gates[t, gate_off + h * dv:gate_off + (h + 1) * dv])
                out[t, h * dv:(h + 1) * dv] = o.to(out.dtype)
        return out

    def conv_silu(self, parts, x_off, channels, weight, bias, conv_state, batch, out):
        x = parts.sum(0)[:, x_off:x_off + channels]
        K = weight.shape[1]
        for s in range(batch.n_seqs):
            first, n, slot = int(batch.seq_qoff[s]), int(batch.seq_ntok[s]), int(batch.seq_slot[s])
            padded = torch.cat([conv_state[slot], x[first:first + n]], dim=0)
            for t in range(n):
                acc = (bias if bias is not None else 0) + (weight.float().t() * padded[t:t + K]).sum(0)
                out[first + t] = torch.nn.functional.silu(acc).to(out.dtype)
            if K > 1:
                conv_state[slot] = padded[padded.shape[0] - (K - 1):]
        return out

    def dt_softplus(self, proj, rank, weight_t, bias, out, n_tokens):
        z = proj[:n_tokens, :rank] @ weight_t.float()
        out[:n_tokens] = torch.nn.functional.softplus(z + bias if bias is not None else z)
        return out

    def selective_scan(self, xc, dt, proj, b_off, c_off, state_size, zparts, z_off, a_log, skip, state, batch, out,
                       dt_bias=None, dt_raw=False):
        A = -torch.exp(a_log)
        C, N = a_log.shape
        z = zparts.sum(0)[:, z_off:z_off + C]
        for s in range(batch.n_seqs):
            first, n, slot = int(batch.seq_qoff[s]), int(batch.seq_ntok[s]), int(batch.seq_slot[s])
            S = state[slot]
            for t in range(first, first + n):
                d = torch.nn.functional.softplus(dt[t] + dt_bias) if dt_raw else dt[t]
                x = xc[t].float()
                S = torch.exp(d[:, None] * A) * S + (d * x)[:, None] * proj[t, b_off:b_off + N][None, :]
                y = S @ proj[t, c_off:c_off + N] + (skip * x if skip is not None else 0)
                out[t] = (y * torch.nn.functional.silu(z[t])).to(out.dtype)
            state[slot] = S
        return out

    # ------------------------------------------------------------------ mixers with a matrix of state per head
    def lowrank_map(self, proj, rank, weight_t, bias, out, n_tokens, in_act=None, out_act="softplus", param=0.0):
        low = proj[:n_tokens, :rank]
        z = (torch.tanh(low) if in_act == "tanh" else low) @ weight_t.float()
        if bias is not None:
            z = z + bias
        if out_act == "sigmoid_root":
            out[:n_tokens] = torch.sigmoid(z) ** (1.0 / param)
        elif out_act == "exp_neg_exp":
            out[:n_tokens] = torch.exp(-torch.exp(z))
        else:
            out[:n_tokens] = torch.nn.functional.softplus(z)
        return out

    def pair_combine(self, a, b, wa, wb, ca, cb, eps, out, n_rows=None):
        n = out.shape[0] if n_rows is None else n_rows
        ys = []
        for t, w in ((a, wa), (b, wb)):
            y = (t if t.dim() == 2 else t.sum(0))[:n]
            if w is not None:
                y = y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * w
            ys.append(y)
        out[:n] = ca * ys[0] + cb * ys[1]
        return out

    def linear_state_shape(self, heads, dk, dv):
        return (heads, dk, dv)

    @staticmethod
    def _cols(t, off, width):
        return (t if t.dim() == 2 else t.sum(0))[:, off:off + width]

    def linear_state(self, rule, q, q_off, k, k_off, v, v_off, decay, decay_off, bonus, state, batch, out, heads, kv_heads, dk, dv,
                     q_scale=1.0, unit_eps=-1.0, decay_const=False):
        Q = self._cols(q, q_off, kv_heads * dk).reshape(-1, kv_heads, dk) * q_scale
        K = self._cols(k, k_off, kv_heads * dk).reshape(-1, kv_heads, dk)
        V = self._cols(v, v_off, heads * dv).reshape(-1, heads, dv)
        if rule == "delta" and unit_eps >= 0:
            Q = Q / torch.sqrt((Q / q_scale).pow(2).sum(-1, keepdim=True) + unit_eps)
            K = K / torch.sqrt(K.pow(2).sum(-1, keepdim=True) + unit_eps)
        rep = heads // kv_heads
        for s in range(batch.n_seqs):
            first, n, slot = int(batch.seq_qoff[s]), int(batch.seq_ntok[s]), int(batch.seq_slot[s])
            S = state[slot].clone()
            for t in range(first, first + n):
                qt, kt, vt = Q[t].repeat_interleave(rep, 0), K[t].repeat_interleave(rep, 0), V[t]
                kv = kt[:, :, None] * vt[:, None, :]
                if rule == "delta":
                    g, beta = decay[t, decay_off:decay_off + heads], decay[t, decay_off + heads:decay_off + 2 * heads]
                    S = S * g[:, None, None]
                    w = beta[:, None] * (vt - torch.einsum("hkv,hk->hv", S, kt))
                    S = S + kt[:, :, None] * w[:, None, :]
                    o = torch.einsum("hkv,hk->hv", S, qt)
                else:
                    a = decay[0 if decay_const else t, decay_off:decay_off + heads * dk].view(heads, dk)
                    if rule == "decay_write_read":
                        S = a[:, :, None] * S + kv
                        o = torch.einsum("hkv,hk->hv", S, qt)
                    else:
                        o = torch.einsum("hkv,hk->hv", S + bonus.view(heads, dk)[:, :, None] * kv, qt)
                        S = a[:, :, None] * S + kv
                out[t] = o.reshape(-1)
            state[slot] = S
        return out

    def rotate_sums(self, x, x_off, heads, dk, cos, sin, positions, out, n_tokens, scaled_from=None, scale=1.0):
        rows = self._cols(x, x_off, heads * dk)[:n_tokens].reshape(n_tokens, heads, dk).clone()
        if cos is not None:
            half = cos.shape[1]
            c, s = cos[positions[:n_tokens].long()][:, None, :], sin[positions[:n_tokens].long()][:, None, :]
            u, v = rows[:, :, :half].clone(), rows[:, :, half:2 * half].clone()
            rows[:, :, :half] = u * c - v * s
            rows[:, :, half:2 * half] = v * c + u * s
        if scaled_from is not None:
            rows[:, scaled_from:] *= scale
        out[:n_tokens] = rows.reshape(n_tokens, heads * dk)
        return out

    def token_shift(self, x, mu, shift_state, batch, out):
        for s in range(batch.n_seqs):
            first, n, slot = int(batch.seq_qoff[s]), int(batch.seq_ntok[s]), int(batch.seq_slot[s])
            if n <= 0:
                continue
            cur = x[first:first + n].float()
            prev = torch.cat([shift_state[slot][None, :], cur[:-1]], dim=0)
            out[:, first:first + n] = (cur[None] + (prev - cur)[None] * mu[:, None, :]).to(out.dtype)
            shift_state[slot] = cur[-1]
        return out

    def delta_gates(self, a, a_off, b, b_off, a_log, dt_bias, out, n_tokens):
        H = a_log.numel()
        za = self._cols(a, a_off, H)[:n_tokens] + dt_bias
        out[:n_tokens, :H] = torch.exp(-torch.exp(a_log) * torch.nn.functional.softplus(za))
        out[:n_tokens, H:] = torch.sigmoid(self._cols(b, b_off, H)[:n_tokens])
        return out

    def head_norm_gate(self, o, weight, gate, gate_off, eps, out, n_tokens, heads, dv):
        y = o[:n_tokens].view(n_tokens, heads, dv)
        y = y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * (weight.view(heads, dv) if weight.numel() == heads * dv and heads > 1 else weight)
        y = y.reshape(n_tokens, heads * dv)
        if gate is not None:
            y = y * torch.nn.functional.silu(self._cols(gate, gate_off, heads * dv)[:n_tokens])
        out[:n_tokens] = y.to(out.dtype)
        return out

    def decode_attention_fusable(self, batch, kcache, nq, nkv, hd, out):
        return False

    def paged_attention(self, q, kcache, vcache, batch, block_table, out, nq, nkv, hd, scale, window=0):
        positions, token_seq, n_tokens = batch.positions, batch.token_seq, batch.n_tokens
        ps = kcache.shape[2]
        g = nq // nkv
        for t in range(n_tokens):
            pos = int(positions[t])
            lo = max(0, pos - window + 1) if window > 0 else 0
            tab = block_table[int(token_seq[t])]
            idx = torch.arange(lo, pos + 1)
            pages = tab[(idx // ps).long()].long()
            assert (pages >= 0).all(), "read from a page that was given back"
            K = kcache[pages, :, (idx % ps).long(), :].float()  # [S, nkv, hd]
            V = vcache[pages, :, (idx % ps).long(), :].float()
            qt = q[t].float().view(nq, hd)
            for h in range(nq):
                s = (K[:, h // g, :] @ qt[h]) * scale
                p = torch.softmax(s, dim=0)
                out[t, h * hd:(h + 1) * hd] = (p @ V[:, h // g, :]).to(out.dtype)
        return out

    @staticmethod
    def _mix32(x):
        x = x.astype(np.uint32)
        x ^= x >> np.uint32(16)
        x = (x * np.uint32(0x7FEB352D)).astype(np.uint32)
        x ^= x >> np.uint32(15)
        x = (x * np.uint32(0x846CA68B)).astype(np.uint32)
        x ^= x >> np.uint32(16)
        return x

    def sample(self, logits, out, temperature=None, seeds=None, draws=None, n_rows=None, scratch=None):
        n = logits.shape[0] if n_rows is None else n_rows
        V = logits.shape[1]
        for r in range(n):
            row = logits[r].float().numpy()
            T = float(temperature[r]) if temperature is not None else 0.0
            if T > 0:
                with np.errstate(over="ignore"):
                    k = self._mix32(np.array([int(seeds[r]) & 0xFFFFFFFF], dtype=np.uint32) ^ np.uint32(0x9E3779B9))
                    k = self._mix32(k + np.uint32(int(draws[r]) & 0xFFFFFFFF))
                    rr = self._mix32(k ^ (np.arange(V, dtype=np.uint32) * np.uint32(0x85EBCA6B)).astype(np.uint32))
                u = ((rr >> np.uint32(9)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 8388608.0)
                gum = -np.log(-np.log(u, dtype=np.float32), dtype=np.float32)
                row = row * (np.float32(1.0) / np.float32(T)) + gum
            out[r] = int(np.argmax(row))
        return out
