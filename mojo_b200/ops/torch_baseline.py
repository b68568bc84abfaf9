"""The same-box baseline: every custom op swapped for stock PyTorch on the GPU (cuBLAS GEMMs through torch.matmul,
scaled_dot_product_attention, eager elementwise kernels), with NCCL collectives from `parallel.tp.NcclTPComm`.
`enable()` rebinds the functions in `mojo_b200.ops`; the engine, scheduler and model code stay identical, so the
ratio product / baseline isolates the kernels."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import ops
from . import reference

_enabled = False


def _rms_norm(x, weight, eps=1e-5, residual=None, out=None):
    if residual is not None:
        residual.add_(x)
        x = residual
    xf = x.float()
    y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(x.dtype)
    return y, x


def _linear(x, w, residual=None, out=None, config=0):
    y = torch.matmul(x, w.t())
    if residual is not None:
        y = y + residual
    return y


def _linear_swiglu(x, w_gu, out=None, config=0):
    y = torch.matmul(x, w_gu.t())
    m = y.shape[0]
    y = y.view(m, -1, 2, 16)
    return (F.silu(y[:, :, 0].float()) * y[:, :, 1].float()).to(x.dtype).reshape(m, -1)


def _rope_kvwrite(q, k, v, cos_sin, positions, slots, k_cache, v_cache, head_dim, interleaved=False):
    T = q.shape[0]
    q.copy_(reference.apply_rope(q.reshape(T, -1, head_dim), positions, cos_sin, interleaved).reshape(T, -1).to(q.dtype))
    k.copy_(reference.apply_rope(k.reshape(T, -1, head_dim), positions, cos_sin, interleaved).reshape(T, -1).to(k.dtype))
    if k_cache is not None:
        page = k_cache.shape[2]
        valid = slots >= 0
        s = slots.clamp_min(0)
        pg, off = s // page, s % page
        kk, vv = k.reshape(T, -1, head_dim), v.reshape(T, -1, head_dim)
        if bool(valid.all()):
            k_cache[pg, :, off] = kk
            v_cache[pg, :, off] = vv
        else:
            k_cache[pg[valid], :, off[valid]] = kk[valid]
            v_cache[pg[valid], :, off[valid]] = vv[valid]


def _paged_attention(q, k_cache, v_cache, meta, scale, head_dim, out=None):
    """Decode rows and prefill chunks as two batched scaled_dot_product_attention calls over K/V gathered through the
    block tables and padded to the longest context / chunk of the step (`meta.max_ctx`, `meta.max_q_len`, both known on
    the host): no per-sequence loop and no device->host synchronisation."""
    T = q.shape[0]
    n_kv, page = k_cache.shape[1], k_cache.shape[2]
    qh = q.reshape(T, -1, head_dim)
    n_q = qh.shape[1]
    # one spare row takes the writes of padding positions
    o = torch.zeros(T + 1, n_q, head_dim, dtype=q.dtype, device=q.device)
    nd, ns = meta.num_decode, meta.num_seqs
    n_pages = max(1, min((max(meta.max_ctx, 1) + page - 1) // page, meta.block_tables.shape[1]))
    kpos = torch.arange(n_pages * page, device=q.device)

    def gather(bt):
        k = k_cache[bt.long()].permute(0, 2, 1, 3, 4).reshape(bt.shape[0], n_kv, -1, head_dim)
        v = v_cache[bt.long()].permute(0, 2, 1, 3, 4).reshape(bt.shape[0], n_kv, -1, head_dim)
        return k, v

    if nd > 0:
        k, v = gather(meta.block_tables[:nd, :n_pages])
        mask = kpos[None, :] < meta.ctx_lens[:nd, None]
        o[:nd] = F.scaled_dot_product_attention(qh[:nd].unsqueeze(2), k, v, attn_mask=mask[:, None, None, :], scale=scale,
                                                enable_gqa=True).squeeze(2)
    if ns > nd:
        P, Lq = ns - nd, max(1, meta.max_q_len)
        cu = meta.cu_q[nd:].long()
        q_len, ctx = cu[1:] - cu[:-1], meta.ctx_lens[nd:].long()
        ar = torch.arange(Lq, device=q.device)
        valid = ar[None, :] < q_len[:, None]                                   # [P, Lq]
        rows = torch.where(valid, cu[:-1, None] + ar[None, :], torch.full_like(valid, T, dtype=torch.long))
        qp = qh[rows.clamp(max=T - 1)].permute(0, 2, 1, 3)                      # [P, heads, Lq, D]
        k, v = gather(meta.block_tables[nd:, :n_pages])
        pos_q = (ctx - q_len)[:, None] + ar[None, :]                            # absolute position of every query row
        mask = kpos[None, None, :] <= pos_q[:, :, None]                         # causal; rows past the chunk see a harmless prefix
        res = F.scaled_dot_product_attention(qp, k, v, attn_mask=mask[:, None], scale=scale, enable_gqa=True)
        o.index_put_((rows.reshape(-1),), res.permute(0, 2, 1, 3).reshape(P * Lq, n_q, head_dim))
    return o[:T].reshape(T, -1)


def enable() -> None:
    """Swap the op table. CUDA-graph capture stays off for this mode (plain eager PyTorch is the point of the arm)."""
    global _enabled
    if _enabled:
        return
    ops.rms_norm = _rms_norm
    ops.linear = _linear
    ops.linear_swiglu = _linear_swiglu
    ops.rope_kvwrite = _rope_kvwrite
    ops.paged_attention = _paged_attention
    ops.embedding = lambda ids, table, vocab_start=0: table[ids]
    ops.gather_rows = lambda src, index: src[index]
    ops.argmax = lambda logits: torch.argmax(logits, dim=-1)
    _enabled = True
