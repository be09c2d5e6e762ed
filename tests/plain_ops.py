"""Plain PyTorch/NumPy statement of every operation in `gpt_fast_b200.ops`.

Two uses.  (1) Each kernel's reference: the GPU tests call a kernel and the
function of the same name here on the same inputs and compare.  (2) A
stand-in for the kernels (`ops.use_kernels(PlainOps())`), so that the host-side
logic of the library (cache, step function, generation loop, replay) can be
exercised on a machine without a GPU.  It is test code: the library itself has
no CPU path.

Accumulations are done in float64, so that the reference is tighter than the
32-bit kernels it judges.
"""
import math

import numpy as np
import torch


def token_positions(batch):
    """Absolute position of every packed token, as the kernels derive it."""
    seq = batch.tok_seq.long()
    slots = batch.slots.long()[seq]
    start = batch.lengths.long()[slots]
    t = torch.arange(batch.n_tokens, device=seq.device)
    return start + (t - batch.cu_seqlens.long()[seq]), slots


# ---- Philox4x32-10, as in csrc/sampling.cu ---------------------------------------
_M0, _M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_MASK = np.uint64(0xFFFFFFFF)


def philox4x32_10(c0, c1, c2, c3, k0, k1):
    c0, c1, c2, c3 = (np.asarray(c, dtype=np.uint64) & _MASK for c in (c0, c1, c2, c3))
    k0, k1 = int(k0) & 0xFFFFFFFF, int(k1) & 0xFFFFFFFF
    for _ in range(10):
        p0, p1 = _M0 * c0, _M1 * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & _MASK
        hi1, lo1 = p1 >> np.uint64(32), p1 & _MASK
        c0, c1, c2, c3 = hi1 ^ c1 ^ np.uint64(k0), lo1, hi0 ^ c3 ^ np.uint64(k1), lo0
        k0, k1 = (k0 + _W0) & 0xFFFFFFFF, (k1 + _W1) & 0xFFFFFFFF
    return c0, c1, c2, c3


def race_noise(seed, request, token_index, V):
    """Exp(1) noise of one row: -log(u), u = ((r >> 9) + 0.5) / 2^23, float32."""
    i = np.arange(V, dtype=np.uint64)
    req = int(request) & (2 ** 64 - 1)
    seed = int(seed) & (2 ** 64 - 1)
    r0, _, _, _ = philox4x32_10(i, np.uint64(int(token_index) & 0xFFFFFFFF), np.uint64(req & 0xFFFFFFFF),
                                np.uint64(req >> 32), seed & 0xFFFFFFFF, seed >> 32)
    u = ((r0 >> np.uint64(9)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 8388608.0)
    return -np.log(u, dtype=np.float32)


class PlainOps:
    # -- element-wise / per-row ---------------------------------------------------
    def softcap(self, x, cap):
        x.copy_((cap * torch.tanh(x.double() / cap)).float())

    def embed(self, tokens, table, out, status, scale=1.0):
        ids = tokens.long()
        bad = (ids < 0) | (ids >= table.shape[0])
        if bad.any():
            t = int(bad.nonzero()[0])
            if status[0] == 0:
                status[0], status[1], status[2] = 1, t, int(ids[t])
        out.copy_(table[ids.clamp(0, table.shape[0] - 1)].float() * scale)
        out[bad] = 0

    def rmsnorm(self, x, weight, eps, out, rows=None, pending=None):
        if pending is not None:
            self.add_partials(x, pending)
        xr = (x if rows is None else x[rows.long()]).double()
        n = xr * torch.rsqrt((xr * xr).mean(-1, keepdim=True) + eps)
        out.copy_((n * weight.double()).to(out.dtype))

    def rope_table(self, inv_freq, table):
        ang = torch.arange(table.shape[0], dtype=torch.float32, device=table.device)[:, None] * inv_freq[None, :]
        table[..., 0] = torch.cos(ang.double()).float()
        table[..., 1] = torch.sin(ang.double()).float()

    def add_partials(self, x, pending):
        x.copy_((x.double() + pending.double().sum(0)).float())

    def rope_append(self, qkv, q_out, kv, batch, table, n_head, n_kv, head_dim, pairing="interleaved", append=True,
                    partials=None):
        H, G, d = n_head, n_kv, head_dim
        T = batch.n_tokens
        if partials is not None:
            qkv = partials.double().sum(0)
        pos, slots = token_positions(batch)
        if int(pos.max()) >= table.shape[0]:
            raise IndexError("position beyond the rotary table")
        cs = table[pos].double()                        # [T, d/2, 2]
        x = qkv.double().view(T, H + 2 * G, d)

        def rotate(v):                                  # v [T, heads, d]
            if pairing == "interleaved":
                a, b = v[..., 0::2], v[..., 1::2]
            else:
                a, b = v[..., : d // 2], v[..., d // 2:]
            c, s = cs[:, None, :, 0], cs[:, None, :, 1]
            oa, ob = a * c - b * s, b * c + a * s
            if pairing == "interleaved":
                return torch.stack([oa, ob], -1).flatten(-2)
            return torch.cat([oa, ob], -1)

        q_out.copy_(rotate(x[:, :H]).to(q_out.dtype))
        if append:
            k = rotate(x[:, H:H + G]).to(kv.k_pool.dtype)
            v = x[:, H + G:].to(kv.v_pool.dtype)
            page = kv.page_table.long()[slots, pos // kv.page_size]
            if int(page.min()) < 0:
                raise IndexError("token lands on a page the slot does not hold")
            off = pos % kv.page_size
            kv.k_pool[page, :, off] = k
            kv.v_pool[page, :, off] = v

    def advance_lengths(self, batch):
        q = (batch.cu_seqlens[1:] - batch.cu_seqlens[:-1]).to(batch.lengths.dtype)
        batch.lengths[batch.slots.long()] += q

    def add_into(self, out, y):
        out += y.float()

    # -- matrix products ---------------------------------------------------------------
    def linear(self, a, w, out, mode="store", defer=False):
        acc = a.double() @ w.double().T
        if mode == "store":
            out.copy_(acc.to(out.dtype))
        elif mode == "add":
            out.copy_((out.double() + acc).to(out.dtype))
        elif mode == "swiglu":
            g, u = acc[:, 0::2], acc[:, 1::2]
            out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))
        else:
            raise ValueError(mode)

    # -- attention -----------------------------------------------------------------------
    def attention(self, q, kv, batch, out, n_head, n_kv, head_dim, scale, window=None):
        H, G, d = n_head, n_kv, head_dim
        pos, slots = token_positions(batch)
        rep = H // G
        res = torch.empty(batch.n_tokens, H, d, dtype=torch.float64, device=q.device)
        for t in range(batch.n_tokens):
            p, slot = int(pos[t]), int(slots[t])
            lo = max(0, p - window + 1) if window else 0
            j = torch.arange(lo, p + 1, device=q.device)
            pages = kv.page_table.long()[slot, j // kv.page_size]
            if int(pages.min()) < 0:
                raise IndexError("attention reads a page the slot does not hold")
            k = kv.k_pool[pages, :, j % kv.page_size].double()      # [n, G, d]
            v = kv.v_pool[pages, :, j % kv.page_size].double()
            k = k.repeat_interleave(rep, dim=1)
            v = v.repeat_interleave(rep, dim=1)
            s = torch.einsum("hd,nhd->hn", q[t].double(), k) * scale
            res[t] = torch.einsum("hn,nhd->hd", torch.softmax(s, -1), v)
        out.copy_(res.view(batch.n_tokens, H * d).to(out.dtype))

    # -- sampling ----------------------------------------------------------------------------
    def argmax(self, logits, out):
        out.copy_(torch.argmax(logits, dim=-1).to(out.dtype))

    def sample(self, logits, out, temperature, top_k, seed, request_ids=None, token_index=None, index_map=None,
               noise_out=None, seed_dev=None):
        if seed_dev is not None:
            seed = int(seed_dev[0])
        B, V = logits.shape
        x = logits.float().cpu() / np.float32(max(temperature, 1e-5))
        for b in range(B):
            row = x[b]
            if top_k and top_k < V:
                pivot = torch.topk(row, top_k).values[-1]
                row = torch.where(row < pivot, torch.tensor(-math.inf), row)
            req = int(request_ids[b]) if request_ids is not None else b
            tix = 0
            if token_index is not None:
                tix = int(token_index[int(index_map[b]) if index_map is not None else b])
            qn = torch.from_numpy(race_noise(seed, req, tix, V))
            if noise_out is not None:
                noise_out[b] = qn.to(noise_out.device)
            score = torch.exp(row - row.max()) / qn
            out[b] = int(torch.argmax(score))
