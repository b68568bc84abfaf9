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
    T = q.shape[0]
    n_kv, page = k_cache.shape[1], k_cache.shape[2]
    qh = q.reshape(T, -1, head_dim)
    o = torch.empty(T, qh.shape[1], head_dim, dtype=q.dtype, device=q.device)
    nd = meta.num_decode
    if nd > 0:
        bt = meta.block_tables[:nd].long()
        k = k_cache[bt].permute(0, 2, 1, 3, 4).reshape(nd, n_kv, -1, head_dim)
        v = v_cache[bt].permute(0, 2, 1, 3, 4).reshape(nd, n_kv, -1, head_dim)
        mask = torch.arange(k.shape[2], device=q.device)[None, :] < meta.ctx_lens[:nd, None]
        o[:nd] = F.scaled_dot_product_attention(qh[:nd].unsqueeze(2), k, v, attn_mask=mask[:, None, None, :], scale=scale,
                                                enable_gqa=True).squeeze(2)
    cu, ctx = meta.cu_q.tolist(), meta.ctx_lens.tolist()
    for b in range(nd, meta.num_seqs):
        s, e, c = cu[b], cu[b + 1], ctx[b]
        n_pages = (c + page - 1) // page
        bt = meta.block_tables[b, :n_pages].long()
        k = k_cache[bt].permute(1, 0, 2, 3).reshape(n_kv, -1, head_dim)[:, :c]
        v = v_cache[bt].permute(1, 0, 2, 3).reshape(n_kv, -1, head_dim)[:, :c]
        ql = e - s
        mask = torch.arange(c, device=q.device)[None, :] <= torch.arange(c - ql, c, device=q.device)[:, None]
        o[s:e] = F.scaled_dot_product_attention(qh[s:e].transpose(0, 1).unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0),
                                                attn_mask=mask, scale=scale, enable_gqa=True)[0].transpose(0, 1)
    return o.reshape(T, -1)


def enable() -> None:
    """Swap the op table. CUDA-graph capture stays off for this mode (the attention fallback syncs)."""
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
