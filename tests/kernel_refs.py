"""Plain torch references for every kernel, with the kernels' own signatures.

Two uses: the ``-m gpu`` tests run each CUDA kernel beside its reference here, and the
CPU tests put this class in the place of the kernel set to exercise the engine's
plumbing (batching, cache, block tables, scheduler) without a GPU.  It is test code
only; the package never imports it.
"""
from __future__ import annotations

import math

import torch

from flint_b200.csrc.ops import MoePlan


def _act(g, name):
    if name == "silu":
        return g / (1.0 + torch.exp(-g))
    if name == "gelu":
        return 0.5 * g * (1.0 + torch.erf(g / math.sqrt(2.0)))
    if name == "none":
        return g
    if name == "relu2":
        return torch.clamp(g, min=0) ** 2
    return 0.5 * g * (1.0 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))


class RefOps:
    name = "reference"

    def __init__(self, compute_dtype=torch.float32):
        self.cd = compute_dtype     # float64 gives an oracle for kernel tests
        self.launches = 0
        # the sampled tokens beside the two error flags, as the device kernels keep them
        self.MAX_TOKEN_ROWS = 256
        self.readback = torch.zeros(2 + self.MAX_TOKEN_ROWS, dtype=torch.int32)
        self.tc_error, self.page_error, self.token_out = self.readback[0:1], self.readback[1:2], self.readback[2:]

    # ------------------------------------------------------------------ row-wise
    def embed(self, ids, table, out, scale=1.0, fed_rows=None, fed_from=None):
        ids = ids.long()
        if fed_rows is not None:
            fed = fed_rows.long()
            ids = torch.where(fed >= 0, fed_from.to(fed.device).long()[fed.clamp(min=0)], ids)
        out.copy_((table[ids].to(self.cd) * scale).to(out.dtype))

    def norm(self, x, gamma, beta, eps, mode, out_f32=None, out_bf16=None, row_index=None):
        xs = x[row_index.long()] if row_index is not None else x
        xs = xs.to(self.cd)
        if mode == "layer":
            mu = xs.mean(-1, keepdim=True)
            var = ((xs - mu) ** 2).mean(-1, keepdim=True)
            y = (xs - mu) / torch.sqrt(var + eps) * gamma.to(self.cd)
            if beta is not None:
                y = y + beta.to(self.cd)
        else:
            y = xs / torch.sqrt((xs ** 2).mean(-1, keepdim=True) + eps) * gamma.to(self.cd)
        if out_f32 is not None:
            out_f32.copy_(y.to(torch.float32))
        if out_bf16 is not None:
            out_bf16.copy_(y.to(torch.float32).to(torch.bfloat16))

    def row_norm(self, x, gamma, beta, eps, mode, out_f32=None, out_bf16=None, row_index=None, pending=None,
                 router=None):
        if pending is not None:
            self.apply_pending(x, pending)
        if gamma is None:
            return
        tmp = out_f32
        if router is not None and tmp is None:
            tmp = torch.empty((x.shape[0], x.shape[1]), dtype=torch.float32)
        self.norm(x, gamma, beta, eps, mode, out_f32=tmp, out_bf16=out_bf16, row_index=row_index)
        if router is not None:
            if getattr(router, "rule", "") == "sigmoid_grouped":
                self.router_sigmoid_grouped(tmp, router.weight, router.correction, router.top, router.groups, router.keep,
                                            router.normalize, router.scale, router.expert_ids, router.gates,
                                            getattr(router, "logits", None))
            elif getattr(router, "rule", "") == "sigmoid":
                self.router_sigmoid(tmp, router.weight, router.weight.shape[0] - router.extra, router.top, router.expert_ids,
                                    router.gates, router.weights, getattr(router, "logits", None))
            elif int(getattr(router, "top", 0)) > 0:
                self.router_topk(tmp, router.weight, router.top, router.groups, router.keep, router.scale,
                                 router.expert_ids, router.gates, getattr(router, "logits", None))
            else:
                self.router_sparsemixer(tmp, router.weight, router.jitter_eps, router.expert_ids, router.gates,
                                        getattr(router, "logits", None))

    def apply_pending(self, x, pending):
        if pending.partials is not None:
            add = pending.partials.to(self.cd).sum(0)
            if pending.bias is not None:
                add = add + pending.bias.to(self.cd)
            x.add_(add.to(x.dtype))
        if pending.y is not None:
            self.moe_combine(x, pending.y, pending.row_of, pending.gates)

    def gemm_partials(self, x, w, splits=None, plan=None):
        out = torch.empty((1, x.shape[0], w.shape[-2]), dtype=torch.float32)
        if plan is None:
            self.gemm(x, w, out[0])
        else:
            self.grouped_gemm(x, w, out[0], plan)
        return out

    def rope_kv_write(self, qkv, pos, slot, cos, sin, rot, q_out, cache, nq, nkv, hd, write_kv, status, bias=None,
                      style="half"):
        if qkv.dim() == 3:
            qkv = qkv.to(self.cd).sum(0)
        if bias is not None:
            qkv = qkv.to(self.cd) + bias.to(self.cd)
        T = qkv.shape[0]
        x = qkv.to(self.cd).view(T, nq + 2 * nkv, hd)
        half = rot // 2
        p = pos.long()

        def rotate(h):
            if rot == 0:
                return h
            c = cos[p].to(self.cd)[:, None, :]
            s = sin[p].to(self.cd)[:, None, :]
            if style == "interleaved":          # dims 2i and 2i + 1 rotate together
                a, b, rest = h[..., 0:rot:2], h[..., 1:rot:2], h[..., rot:]
                both = torch.stack([a * c - b * s, b * c + a * s], -1).reshape(*h.shape[:-1], rot)
                return torch.cat([both, rest], -1)
            a, b, rest = h[..., :half], h[..., half:rot], h[..., rot:]
            return torch.cat([a * c - b * s, b * c + a * s, rest], -1)
        q_out.copy_(rotate(x[:, :nq]).reshape(T, nq * hd).to(q_out.dtype))
        if not write_kv:
            return
        k = rotate(x[:, nq:nq + nkv])
        v = x[:, nq + nkv:]
        P = cache.page_size
        pages = cache.block_table[slot.long(), (p // P)].long()
        assert (pages >= 0).all(), "write to a position without a page"
        cache.k[pages, :, p % P, :] = k.to(cache.k.dtype)
        cache.v[pages, :, p % P, :] = v.to(cache.v.dtype)

    def gather_rows(self, x, index, out):
        idx = index.long()
        rows = x[idx.clamp(min=0)].clone()
        rows[idx < 0] = 0
        out.copy_(rows)

    def moe_combine(self, h, y, row_of, gates):
        k = row_of.numel() // h.shape[0]
        r = row_of.view(-1, k).long()
        g = gates.view(-1, k).to(self.cd)
        yy = y.to(self.cd)
        h.add_(sum(g[:, i:i + 1] * yy[r[:, i]] for i in range(k)).to(h.dtype))

    # ------------------------------------------------------------------ matrix products
    def gemm(self, x, w, out, bias=None, accumulate=False):
        y = x.to(self.cd) @ w.to(self.cd).T
        if bias is not None:
            y = y + bias.to(self.cd)
        if accumulate:
            y = y + out.to(self.cd)
        out.copy_(y.to(out.dtype))

    def _rows_by_expert(self, plan):
        off = plan.offsets.tolist()
        return [(e, off[e], off[e + 1]) for e in range(plan.n_experts) if off[e + 1] > off[e]]

    @staticmethod
    def pair_gate_up(w_gate, w_up):
        """This implementation keeps the gate rows before the up rows."""
        return torch.cat([w_gate, w_up], -2)

    def gated_gemm(self, x, w13, out, act="silu", plan=None, act_params=None):
        """w13 = pair_gate_up(gate, up): [2N, K] or [E, 2N, K]."""
        xs = x.to(self.cd)
        n = w13.shape[-2] // 2
        if act == "swish_clamped":
            slope, limit = act_params
            g = torch.clamp(xs @ w13[:n].to(self.cd).T, max=limit)
            u = torch.clamp(xs @ w13[n:].to(self.cd).T, -limit, limit)
            out.copy_((g * torch.sigmoid(slope * g) * (u + 1.0)).to(out.dtype))
            return
        if plan is None:
            out.copy_((_act(xs @ w13[:n].to(self.cd).T, act) * (xs @ w13[n:].to(self.cd).T)).to(out.dtype))
            return
        for e, lo, hi in self._rows_by_expert(plan):
            g = xs[lo:hi] @ w13[e, :n].to(self.cd).T
            u = xs[lo:hi] @ w13[e, n:].to(self.cd).T
            out[lo:hi] = (_act(g, act) * u).to(out.dtype)

    def grouped_gemm(self, x, w, out, plan, plan_ready=False):
        xs = x.to(self.cd)
        for e, lo, hi in self._rows_by_expert(plan):
            out[lo:hi] = (xs[lo:hi] @ w[e].to(self.cd).T).to(out.dtype)

    # ------------------------------------------------------------------ attention
    def attention(self, q, cache, step, out, nq, nkv, hd, window, scale, tiling=None):
        self.paged_attention(q, cache, step.pos, step.slot, out, nq, nkv, hd, window, scale, step.max_kv_len)

    def paged_attention(self, q, cache, pos, slot, out, nq, nkv, hd, window, scale, max_kv_len, splits=None,
                        kernel=None, rows=None):
        T = q.shape[0]
        P = cache.page_size
        G = nq // nkv
        qq = q.to(self.cd).view(T, nq, hd)
        res = out.to(self.cd).view(T, nq, hd).clone()
        for t in (range(T) if rows is None else rows.tolist()):
            p = int(pos[t])
            lo = max(0, p + 1 - window) if window else 0
            js = torch.arange(lo, p + 1)
            pages = cache.block_table[int(slot[t]), js // P].long()
            assert (pages >= 0).all(), f"row {t}: key without a page"
            k = cache.k[pages, :, js % P, :].to(self.cd)      # [n, nkv, hd]
            v = cache.v[pages, :, js % P, :].to(self.cd)
            for h in range(nq):
                s = (k[:, h // G, :] @ qq[t, h]) * scale
                res[t, h] = torch.softmax(s, 0) @ v[:, h // G, :]
        out.copy_(res.reshape(T, nq * hd).to(out.dtype))

    def moe_tile_rows(self, n_tokens, n_experts, weight_dtype, top=2):
        return 64

    # ------------------------------------------------------------------ attention with kept first tokens and a sink
    def qkv_write(self, qkv, bias, pos, slot, cos, sin, rot, style, q_out, cache, nq, nkv, hd, vd, status,
                  v_keep=None, v_from=None, blend=0.0):
        x = qkv.to(self.cd).sum(0) if qkv.dim() == 3 else qkv.to(self.cd)
        if bias is not None:
            x = x + bias.to(self.cd)
        T = x.shape[0]
        p = pos.long()
        half = rot // 2

        def rotate(h):
            if rot == 0:
                return h
            c, s_ = cos[p].to(self.cd)[:, None, :], sin[p].to(self.cd)[:, None, :]
            if style == "interleaved":
                a, b = h[..., 0:rot:2], h[..., 1:rot:2]
                both = torch.stack([a * c - b * s_, b * c + a * s_], -1).reshape(*h.shape[:-1], rot)
            else:
                a, b = h[..., :half], h[..., half:rot]
                both = torch.cat([a * c - b * s_, b * c + a * s_], -1)
            return torch.cat([both, h[..., rot:]], -1)
        q = rotate(x[:, :nq * hd].view(T, nq, hd))
        k = rotate(x[:, nq * hd:(nq + nkv) * hd].view(T, nkv, hd))
        v = x[:, (nq + nkv) * hd:].view(T, nkv, vd)
        if v_keep is not None:
            v_keep.copy_(v.reshape(T, nkv * vd).to(v_keep.dtype))
        if v_from is not None:
            v = (1.0 - blend) * v + blend * v_from.to(self.cd).view(T, nkv, vd)
        q_out.copy_(q.reshape(T, nq * hd).to(q_out.dtype))
        P = cache.page_size
        pages = cache.block_table[slot.long(), p // P].long()
        assert (pages >= 0).all(), "write to a position without a page"
        cache.k[pages, :, p % P, :] = k.to(cache.k.dtype)
        cache.v[pages, :, p % P, :] = v.to(cache.v.dtype)

    def sink_attention(self, q, cache, step, out, nq, nkv, hd, vd, window, keep_first, sinks, scale, splits=None,
                       tiling=None, rows=None, chunk=0, pool=0, sigmoid=None):
        T, P, G = q.shape[0], cache.page_size, nq // nkv
        qq = q.to(self.cd).view(T, nq, hd)
        res = torch.zeros(T, nq, vd, dtype=self.cd)
        for t in range(T):
            p = int(step.pos[t])
            lo = max(0, p + 1 - window) if window else 0
            if chunk:
                lo = (p // chunk) * chunk
            js = torch.cat([torch.arange(0, min(keep_first, lo)), torch.arange(lo, p + 1)])
            pages = cache.block_table[int(step.slot[t]), js // P].long()
            assert (pages >= 0).all(), f"row {t}: key without a page"
            k = cache.k[pages, :, js % P, :].to(self.cd)
            v = cache.v[pages, :, js % P, :].to(self.cd)
            if pool and p - window + 1 >= pool:        # the means of the blocks that lie wholly before the window
                bs = torch.arange((p - window + 1) // pool)
                E = cache.pool_slots
                homes = cache.block_table[int(step.slot[t]), bs // E].long()
                assert (homes >= 0).all(), f"row {t}: block mean without a page"
                k = torch.cat([cache.pool_k[homes, :, bs % E, :].to(self.cd), k], 0)
                v = torch.cat([cache.pool_v[homes, :, bs % E, :].to(self.cd), v], 0)
            for h in range(nq):
                s = (k[:, h // G, :] @ qq[t, h]) * scale
                if sigmoid is not None:
                    cap, r1, r2, bias = sigmoid
                    if cap:
                        s = cap * torch.tanh(s / cap)
                    if r1 is not None:
                        s = s - r1[h].to(self.cd) * torch.log(1 + r2[h].to(self.cd) * (p - js).to(self.cd))
                    if bias is not None:
                        s = s + bias[h].to(self.cd)
                    res[t, h] = torch.sigmoid(s) @ v[:, h // G, :]
                    continue
                if sinks is not None:
                    s = torch.cat([s, sinks[h].to(self.cd).view(1)])
                w = torch.softmax(s, 0)[:k.shape[0]]
                res[t, h] = w @ v[:, h // G, :]
        out.copy_(res.reshape(T, nq * vd).to(out.dtype))

    # ------------------------------------------------------------------ matrix memory
    def mlstm_scan(self, proj, b_gates, slot, seq_start, n_seq, state, out, H, D, V, cap):
        x = proj.to(self.cd).sum(0) if proj.dim() == 3 else proj.to(self.cd)
        T = x.shape[0]
        o_q, o_k, o_v, o_g, o_i = 0, H * D, 2 * H * D, 2 * H * D + H * V, 2 * H * D + 2 * H * V
        q = x[:, o_q:o_k].view(T, H, D) * D ** -0.5
        k = x[:, o_k:o_v].view(T, H, D)
        v = x[:, o_v:o_g].view(T, H, V)
        zi = x[:, o_i:o_i + H] + b_gates[:H].to(self.cd)
        zf = x[:, o_i + H:o_i + 2 * H] + b_gates[H:].to(self.cd)
        gi = cap * torch.tanh(zi / cap)
        gf = torch.nn.functional.logsigmoid(cap * torch.tanh(zf / cap))
        starts = list(range(n_seq + 1)) if seq_start is None else seq_start.tolist()
        per = D * V + D + 1
        res = torch.zeros(T, H, V, dtype=self.cd)
        for e in range(n_seq):
            sl = int(slot[starts[e]])
            st = state[sl].to(self.cd).clone()
            for h in range(H):
                S = st[h * per:h * per + D * V].view(V, D).T.clone()
                n = st[h * per + D * V:h * per + D * V + D].clone()
                m = st[h * per + D * V + D].clone()
                for t in range(starts[e], starts[e + 1]):
                    m_new = torch.maximum(gf[t, h] + m, gi[t, h])
                    a, b = torch.exp(gf[t, h] + m - m_new), torch.exp(gi[t, h] - m_new)
                    S = a * S + b * torch.outer(k[t, h], v[t, h])
                    n = a * n + b * k[t, h]
                    m = m_new
                    res[t, h] = (S.T @ q[t, h]) / (torch.maximum(torch.abs(n @ q[t, h]), torch.exp(-m)) + 1e-6)
                st[h * per:h * per + D * V] = S.T.reshape(-1)
                st[h * per + D * V:h * per + D * V + D] = n
                st[h * per + D * V + D] = m
            state[sl] = st.to(state.dtype)
        out.copy_(res.reshape(T, H * V).to(out.dtype))
        return x[:, o_g:o_i].to(torch.float32)

    def mlstm_finish(self, o, gate, norm_w, eps, out, H, V):
        T = o.shape[0]
        x = o.to(self.cd).view(T, H, V)
        x = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
        y = x.reshape(T, H * V) * norm_w.to(self.cd) * torch.sigmoid(gate.to(self.cd))
        out.copy_(y.to(out.dtype))

    # ------------------------------------------------------------------ state carried from token to token
    @staticmethod
    def _runs(pos, slot):
        """[(first row, one past the last row)] of every request's rows in the batch."""
        T, runs, a = pos.numel(), [], 0
        for t in range(1, T + 1):
            if t == T or int(slot[t]) != int(slot[t - 1]) or int(pos[t]) != int(pos[t - 1]) + 1:
                runs.append((a, t))
                a = t
        return runs

    def short_conv(self, u, col0, w, bias, act, pos, slot, state, y):
        C, taps = w.shape
        x = u[:, col0:col0 + C].to(self.cd)
        ww = w.to(self.cd)
        res = torch.zeros(x.shape, dtype=self.cd)
        for a, b in self._runs(pos, slot):
            sl, p0 = int(slot[a]), int(pos[a])
            past = torch.zeros(taps - 1, C, dtype=self.cd)       # inputs of positions p0 - taps + 1 .. p0 - 1
            for d in range(1, taps):
                if p0 - d >= 0:
                    r = (p0 - d) % (taps - 1)
                    past[taps - 1 - d] = state[sl, r * C:(r + 1) * C].to(self.cd)
            seq = torch.cat([past, x[a:b]], 0)
            for j in range(taps):
                res[a:b] += ww[:, j] * seq[j:j + b - a]
            for t in range(max(a, b - (taps - 1)), b):
                r = int(pos[t]) % (taps - 1)
                state[sl, r * C:(r + 1) * C] = x[t].to(state.dtype)
        if bias is not None:
            res = res + bias.to(self.cd)
        y.copy_(_act(res, act).to(y.dtype))

    def delta_prepare(self, y, b, a, dt_bias, a_log, qk, decay, beta, H, G, D, unit_eps):
        T = y.shape[0]
        x = y[:, :2 * G * D].to(self.cd).view(T, 2 * G, D)
        x = x / torch.sqrt((x * x).sum(-1, keepdim=True) + unit_eps)
        x[:, :G] = x[:, :G] * D ** -0.5
        qk.copy_(x.reshape(T, 2 * G * D).to(qk.dtype))
        beta.copy_(torch.sigmoid(b.to(self.cd)).to(beta.dtype))
        sp = torch.nn.functional.softplus(a.to(self.cd) + dt_bias.to(self.cd), threshold=30.0).view(T, H, D)
        decay.copy_(torch.exp(-torch.exp(a_log.to(self.cd)).view(1, H, 1) * sp).reshape(T, H * D).to(decay.dtype))

    def ssd_prepare(self, raw, dt_bias, a_log, dt, decay):
        d = torch.nn.functional.softplus(raw.to(self.cd) + dt_bias.to(self.cd), threshold=30.0)
        dt.copy_(d.to(dt.dtype))
        decay.copy_(torch.exp(-torch.exp(a_log.to(self.cd)) * d).to(decay.dtype))

    def recurrence_scan(self, q, k, v, decay, delta, beta, dt, skip, slot, seq_start, n_seq, state, out, H, G, D, V):
        T = q.shape[0]
        qq, kk, vv = q.to(self.cd).view(T, G, D), k.to(self.cd).view(T, G, D), v.to(self.cd).view(T, H, V)
        dec = decay.to(self.cd).view(T, H, D) if delta else decay.to(self.cd)
        starts = list(range(n_seq + 1)) if seq_start is None else seq_start.tolist()
        res = torch.zeros(T, H, V, dtype=self.cd)
        for e in range(n_seq):
            if starts[e + 1] <= starts[e]:
                continue
            sl = int(slot[starts[e]])
            S = state[sl, :H * D * V].to(self.cd).view(H, D, V).clone()
            for t in range(starts[e], starts[e + 1]):
                for h in range(H):
                    g = h // (H // G)
                    if delta:
                        S[h] = dec[t, h][:, None] * S[h]
                        u = beta[t, h].to(self.cd) * (vv[t, h] - S[h].T @ kk[t, g])
                    else:
                        S[h] = dec[t, h] * S[h]
                        u = dt[t, h].to(self.cd) * vv[t, h]
                    S[h] = S[h] + torch.outer(kk[t, g], u)
                    res[t, h] = S[h].T @ qq[t, g]
                    if skip is not None:
                        res[t, h] = res[t, h] + skip[h].to(self.cd) * vv[t, h]
            state[sl, :H * D * V] = S.reshape(-1).to(state.dtype)
        out.copy_(res.reshape(T, H * V).to(out.dtype))

    def gated_norm(self, o, gate, gate_act, gate_first, w, eps, groups, out):
        T, N = o.shape
        x = o.to(self.cd)
        g = gate.to(self.cd)
        g = g / (1.0 + torch.exp(-g)) if gate_act == "silu" else torch.sigmoid(g)
        if gate_first:
            x = x * g
        x = x.view(T, groups, N // groups)
        x = (x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)).reshape(T, N)
        x = x * w.to(self.cd).repeat(N // w.numel())
        if not gate_first:
            x = x * g
        out.copy_(x.to(out.dtype))

    def branch_mean(self, branches, weights, eps, out):
        acc = torch.zeros(out.shape, dtype=self.cd)
        for (part, bias), w in zip(branches, weights):
            y = part.to(self.cd).sum(0)
            if bias is not None:
                y = y + bias.to(self.cd)
            acc += y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * w.to(self.cd)
        out.copy_((acc / len(branches)).to(out.dtype))

    def post_norm(self, x, partials, bias, scale, residual_scale, gamma, beta, eps, mode, out_copy=None):
        y = partials.to(self.cd).sum(0)
        if bias is not None:
            y = y + bias.to(self.cd)
        if scale is not None:
            y = y * scale.to(self.cd)
        v = residual_scale * x.to(self.cd) + y
        if mode == "layer":
            v = v - v.mean(-1, keepdim=True)
        v = v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * gamma.to(self.cd)
        if beta is not None:
            v = v + beta.to(self.cd)
        x.copy_(v.to(x.dtype))
        if out_copy is not None:
            out_copy.copy_(v.to(torch.float32).to(out_copy.dtype))

    def depth_mix(self, history, n, w, h, out_copy=None):
        history[n - 1].copy_(h)
        acc = (history[:n].to(self.cd) * w[:n].to(self.cd).view(n, 1, 1)).sum(0)
        h.copy_(acc.to(h.dtype))
        if out_copy is not None:
            out_copy.copy_(acc.to(torch.float32).to(out_copy.dtype))

    def softcap(self, x, cap):
        x.copy_((cap * torch.tanh(x.to(self.cd) / cap)).to(x.dtype))

    def cast_rows(self, x, out):
        out.copy_(x.to(out.dtype))

    @staticmethod
    def _turn(h, cos, sin, style, sign=1.0):
        """h [T, heads, n] with the leading 2 * cos.shape[-1] dims rotated by the angles of cos, sin [T, n / 2]."""
        rot = 2 * cos.shape[-1]
        if rot == 0:
            return h
        c, s_ = cos[:, None, :], sign * sin[:, None, :]
        if style == "interleaved":
            a, b = h[..., 0:rot:2], h[..., 1:rot:2]
            both = torch.stack([a * c - b * s_, b * c + a * s_], -1).reshape(*h.shape[:-1], rot)
        else:
            a, b = h[..., :rot // 2], h[..., rot // 2:rot]
            both = torch.cat([a * c - b * s_, b * c + a * s_], -1)
        return torch.cat([both, h[..., rot:]], -1)

    def qk_norm_write(self, y, q_norm, k_norm, eps, pos, slot, cos, sin, rot, style, v_cos, v_sin, v_style, q_out, cache,
                      nq, nkv, hd, vd, status, whole=False, v_from_k=False, q_temp=None):
        T = y.shape[0]
        x = y.to(self.cd)
        p = pos.long()
        q = x[:, :nq * hd].reshape(T, nq, hd)
        k = x[:, nq * hd:(nq + nkv) * hd].reshape(T, nkv, hd)
        v = k.clone() if v_from_k else x[:, (nq + nkv) * hd:(nq + nkv) * hd + nkv * vd].reshape(T, nkv, vd)
        if q_norm is not None and whole:
            q = (q / torch.sqrt((q * q).mean((-2, -1), keepdim=True) + eps)) * q_norm.to(self.cd).view(nq, hd)
            k = (k / torch.sqrt((k * k).mean((-2, -1), keepdim=True) + eps)) * k_norm.to(self.cd).view(nkv, hd)
        elif q_norm is not None:
            q = q / torch.sqrt((q * q).mean(-1, keepdim=True) + eps) * q_norm.to(self.cd)
            k = k / torch.sqrt((k * k).mean(-1, keepdim=True) + eps) * k_norm.to(self.cd)
        if q_temp is not None:
            temp = 1 + q_temp[0] * torch.log(torch.floor((p.to(self.cd) + 1) / q_temp[1]) + 1)
            q = q * temp[:, None, None]
        if rot:
            q = self._turn(q, cos[p].to(self.cd), sin[p].to(self.cd), style)
            k = self._turn(k, cos[p].to(self.cd), sin[p].to(self.cd), style)
        if v_cos is not None:
            v = self._turn(v, v_cos[p].to(self.cd), v_sin[p].to(self.cd), v_style)
        q_out.copy_(q.reshape(T, nq * hd).to(q_out.dtype))
        P = cache.page_size
        pages = cache.block_table[slot.long(), p // P].long()
        assert (pages >= 0).all(), "write to a position without a page"
        cache.k[pages, :, p % P, :] = k.to(cache.k.dtype)
        cache.v[pages, :, p % P, :] = v.to(cache.v.dtype)

    def head_finish(self, attn, pos, v_cos, v_sin, v_style, gate, out, nq, vd):
        T = attn.shape[0]
        x = attn.to(self.cd).view(T, nq, vd)
        if v_cos is not None:
            p = pos.long()
            x = self._turn(x, v_cos[p].to(self.cd), v_sin[p].to(self.cd), v_style, sign=-1.0)
        if gate is not None and gate.shape[1] == nq * vd and vd > 1:
            x = x * torch.sigmoid(gate.to(self.cd)).view(T, nq, vd)
        elif gate is not None:
            x = x * torch.sigmoid(gate.to(self.cd))[:, :, None]
        out.copy_(x.reshape(T, nq * vd).to(out.dtype))

    # ------------------------------------------------------------------ means of blocks, weighted sums, retention, grouped sigmoid router
    def pool_write(self, cache, step, nkv, hd, vd, pool):
        P, E = cache.page_size, cache.pool_slots
        for t in range(step.n_tokens):
            p, sl = int(step.pos[t]), int(step.slot[t])
            if (p + 1) % pool:
                continue
            b = (p + 1) // pool - 1
            js = torch.arange(b * pool, p + 1)
            pages = cache.block_table[sl, js // P].long()
            assert (pages >= 0).all(), "a block's position without a page"
            home = int(cache.block_table[sl, b // E])
            assert home >= 0
            cache.pool_k[home, :, b % E, :] = cache.k[pages, :, js % P, :].to(self.cd).mean(0).to(cache.pool_k.dtype)
            cache.pool_v[home, :, b % E, :] = cache.v[pages, :, js % P, :].to(self.cd).mean(0).to(cache.pool_v.dtype)

    def sum_norm_add(self, dst, branches=(), scales=(), expert_rows=None, gamma=None, eps=0.0, accumulate=True):
        r = torch.zeros(dst.shape, dtype=self.cd)
        for (part, bias), sc in zip(branches, scales):
            y = part.to(self.cd).sum(0)
            if bias is not None:
                y = y + bias.to(self.cd)
            r = r + sc * y
        if expert_rows is not None:
            y, row_of, gates = expert_rows
            r = r + (y.to(self.cd)[row_of.long()] * gates.to(self.cd)[:, :, None]).sum(1)
        if gamma is not None:
            r = r / torch.sqrt((r * r).mean(-1, keepdim=True) + eps) * gamma.to(self.cd)
        dst.copy_(((dst.to(self.cd) if accumulate else 0) + r).to(dst.dtype))

    def retention_prepare(self, proj, pos, cos, sin, rot, style, decay_h, dt_value, qk, decay, dt, H, D):
        T = proj.shape[0]
        x = proj[:, :2 * H * D].to(self.cd).reshape(T, 2 * H, D)
        if rot:
            p = pos.long()
            x = self._turn(x, cos[p].to(self.cd), sin[p].to(self.cd), style)
        qk.copy_(x.reshape(T, 2 * H * D).to(qk.dtype))
        decay.copy_(decay_h.to(decay.dtype)[None, :].expand(T, H))
        dt.fill_(dt_value)

    def router_sigmoid_grouped(self, x, wr, correction, top, n_groups, keep, normalize, scale, expert_ids, gates,
                               logits_out=None):
        z = x.to(self.cd) @ wr.to(self.cd).T
        T, E = z.shape
        s = torch.sigmoid(z)
        c = s + correction.to(self.cd) if correction is not None else s.clone()
        per = E // n_groups
        if keep < n_groups:
            gs = c.view(T, n_groups, per).topk(min(2, per), -1).values.sum(-1)
            order = torch.sort(gs, dim=-1, descending=True, stable=True).indices[:, :keep]
            kept = torch.zeros((T, n_groups), dtype=torch.bool).scatter_(1, order, True)
            c = c.masked_fill(~kept[:, :, None].expand(T, n_groups, per).reshape(T, E), -math.inf)
        idx = torch.sort(c, dim=-1, descending=True, stable=True).indices[:, :top]
        val = s.gather(1, idx)
        if normalize:
            val = val / (val.sum(-1, keepdim=True) + 1e-20)
        expert_ids.copy_(idx.to(torch.int32))
        gates.copy_((val * scale).to(gates.dtype))
        if logits_out is not None:
            logits_out.copy_(z.to(logits_out.dtype))

    # ------------------------------------------------------------------ sigmoid router, plain experts
    def router_sigmoid(self, x, wr, E, top, expert_ids, scores, weights, logits_out=None):
        z = x.to(self.cd) @ wr.to(self.cd).T
        s = torch.sigmoid(z)
        val, idx = torch.sort(s[:, :E], dim=-1, descending=True, stable=True)
        expert_ids.copy_(idx[:, :top].to(torch.int32))
        scores.copy_(val[:, :top].to(scores.dtype))
        weights[:, :top] = 1.0
        if wr.shape[0] > E:
            weights[:, top:] = s[:, E:].to(weights.dtype)
        if logits_out is not None:
            logits_out.copy_(z.to(logits_out.dtype))

    def row_act(self, partials, out, act, row_of=None, row_scale=None):
        x = partials.to(self.cd).sum(0) if partials.dim() == 3 else partials.to(self.cd)
        if row_of is not None:
            scale = torch.ones(x.shape[0], dtype=self.cd)
            scale[row_of.reshape(-1).long()] = row_scale.reshape(-1).to(self.cd)
            x = x * scale[:, None]
        out.copy_(_act(x, act).to(out.dtype))

    # ------------------------------------------------------------------ attention over a cached latent
    def head_products(self, x, w, out):
        out.copy_(torch.einsum("thk,hnk->thn", x.to(self.cd), w.to(self.cd)).to(out.dtype))

    def latent_prepare(self, proj, pos, slot, cos, sin, rot_dims, style, norm_w, eps, q_plain, qa, cache, H, D, R, C,
                       write_kv, status):
        x = (proj.to(self.cd).sum(0) if proj.dim() == 3 else proj.to(self.cd))
        T = x.shape[0]
        p = pos.long()
        half = rot_dims // 2

        def rotate(v):          # [T, ..., R]
            if rot_dims == 0:
                return v
            shape = [T] + [1] * (v.dim() - 2) + [half]
            c, s_ = cos[p].to(self.cd).view(shape), sin[p].to(self.cd).view(shape)
            if style == "interleaved":
                a, b = v[..., 0:rot_dims:2], v[..., 1:rot_dims:2]
                both = torch.stack([a * c - b * s_, b * c + a * s_], -1).reshape(*v.shape[:-1], rot_dims)
            else:
                a, b = v[..., :half], v[..., half:rot_dims]
                both = torch.cat([a * c - b * s_, b * c + a * s_], -1)
            return torch.cat([both, v[..., rot_dims:]], -1)
        q = x[:, :H * (D + R)].view(T, H, D + R)
        q_plain.copy_(q[..., :D].to(q_plain.dtype))
        qa[..., C:] = rotate(q[..., D:]).to(qa.dtype)
        if not write_kv:
            return
        lat = x[:, H * (D + R):]
        c = lat[:, :C]
        c = c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * norm_w.to(self.cd)
        row = torch.zeros(T, cache.k.shape[-1], dtype=self.cd)
        row[:, :C] = c
        row[:, C:C + R] = rotate(lat[:, C:C + R])
        P = cache.page_size
        pages = cache.block_table[slot.long(), p // P].long()
        assert (pages >= 0).all(), "write to a position without a page"
        cache.k[pages, 0, p % P, :] = row.to(cache.k.dtype)

    def latent_attention(self, qa, cache, step, out, H, C, window, scale, splits=None, rows=None):
        T, Dk = qa.shape[0], qa.shape[2]
        P = cache.page_size
        for t in (range(T) if rows is None else rows.tolist()):
            p = int(step.pos[t])
            lo = max(0, p + 1 - window) if window else 0
            js = torch.arange(lo, p + 1)
            pages = cache.block_table[int(step.slot[t]), js // P].long()
            assert (pages >= 0).all(), f"row {t}: key without a page"
            k = cache.k[pages, 0, js % P, :].to(self.cd)            # [n, row]
            s = (qa[t].to(self.cd) @ k[:, :Dk].T) * scale            # [H, n]
            out[t] = (torch.softmax(s, -1) @ k[:, :C]).to(out.dtype)

    def pair_embed_add(self, ids, pos, slot, last, table, out, mul_prev, mul_cur, fed_rows=None, fed_from=None):
        ids = ids.long().clone()
        if fed_rows is not None:
            fed = fed_rows.long()
            ids = torch.where(fed >= 0, fed_from.long()[fed.clamp(min=0)], ids)
        buckets = table.shape[0] - 1
        T = ids.numel()
        rows = []
        for r in range(T):
            if int(pos[r]) == 0:
                rows.append(buckets)
                continue
            first = r == 0 or int(slot[r - 1]) != int(slot[r])
            prev = int(last[int(slot[r])]) if first else int(ids[r - 1])
            rows.append((prev * mul_prev + int(ids[r]) * mul_cur) % buckets)
        out.add_(table[torch.tensor(rows, dtype=torch.long)].to(self.cd).to(out.dtype))
        for r in range(T):
            if r == T - 1 or int(slot[r + 1]) != int(slot[r]):
                last[int(slot[r])] = int(ids[r])

    def router_topk(self, x, wr, top, n_groups, keep, scale, expert_ids, gates, logits_out=None):
        z = x.to(self.cd) @ wr.to(self.cd).T
        if logits_out is not None:
            logits_out.copy_(z.to(logits_out.dtype))
        E = wr.shape[0]
        per = E // n_groups
        for t in range(x.shape[0]):
            s = torch.softmax(z[t], -1)
            allowed = torch.zeros(E, dtype=torch.bool)
            gs = s.view(n_groups, per).max(-1).values.clone()
            for _ in range(keep):
                g = int(torch.argmax(gs))
                allowed[g * per:(g + 1) * per] = True
                gs[g] = -1.0
            cand = s.masked_fill(~allowed, -1.0)
            chosen = []
            for _ in range(top):
                e = int(torch.argmax(cand))
                chosen.append(e)
                cand[e] = -1.0
            w = s[chosen]
            expert_ids[t] = torch.tensor(chosen, dtype=torch.int32)
            gates[t] = (w / (w.sum() + 1e-20) * scale).to(gates.dtype)

    # ------------------------------------------------------------------ routing
    def router_sparsemixer(self, x, wr, eps, expert_ids, gates, logits_out=None):
        s_all = x.to(self.cd) @ wr.to(self.cd).T
        if logits_out is not None:
            logits_out.copy_(s_all.to(logits_out.dtype))
        for t in range(x.shape[0]):
            s = s_all[t]
            excluded = -1
            for r in range(2):
                cand = s.clone()
                if excluded >= 0:
                    cand[excluded] = float("-inf")
                m = cand.max()
                im = int(torch.argmax(cand))
                factor = torch.clamp(s.abs(), min=m)
                masked = ((m - s) / factor) > 2.0 * eps
                masked_scores = cand.masked_fill(masked, float("-inf"))
                expert_ids.view(-1, 2)[t, r] = im
                gates.view(-1, 2)[t, r] = torch.softmax(masked_scores, 0)[im].to(gates.dtype)
                excluded = im

    def moe_plan(self, expert_ids, n_experts, tile_rows):
        ids = expert_ids.reshape(-1).long()
        n = ids.numel()
        counts = torch.bincount(ids, minlength=n_experts)
        offsets = torch.zeros(n_experts + 1, dtype=torch.long)
        offsets[1:] = torch.cumsum(counts, 0)
        order = torch.argsort(ids, stable=True)
        row_of = torch.empty(n, dtype=torch.long)
        row_of[order] = torch.arange(n)
        token_of = order // (expert_ids.shape[-1] if expert_ids.dim() > 1 else 2)
        tiles_e, tiles_r = [], []
        for e in range(n_experts):
            for r in range(0, int(counts[e]), tile_rows):
                tiles_e.append(e)
                tiles_r.append(int(offsets[e]) + r)
        max_tiles = n // tile_rows + min(n_experts, n)
        i32 = lambda t: torch.as_tensor(t, dtype=torch.int32)
        pad = lambda l: i32(l + [0] * (max_tiles - len(l)))
        top = expert_ids.shape[-1] if expert_ids.dim() > 1 else 2
        return MoePlan(n_experts, tile_rows, max_tiles, i32(counts), i32(offsets), i32(row_of).view(-1, top),
                       i32(token_of), pad(tiles_e), pad(tiles_r), i32([len(tiles_e)]), top)

    def moe_dispatch(self, expert_ids, n_experts, tile_rows, x):
        plan = self.moe_plan(expert_ids, n_experts, tile_rows)
        return plan, x[plan.token_of.long()].clone()

    # ------------------------------------------------------------------ sampling
    def argmax(self, logits, out):
        out.copy_(torch.argmax(logits, dim=-1).to(torch.int32))
