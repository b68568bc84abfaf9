"""Op library. Every function takes CUDA bf16 tensors and launches a hand-written sm_100a kernel; given CPU
tensors it evaluates the fp32 reference in `ops.reference` instead (the oracle, and the CPU engine's compute).
There is no other dispatch: a CUDA tensor without the built extension is an ImportError, never a quiet
PyTorch fallback.
"""
from __future__ import annotations

import torch

from .. import _ext
from . import _state, autotune, reference
from ._state import KernelError, check_status

EPI_NONE, EPI_ADD_RESIDUAL, EPI_SWIGLU = 0, 1, 2

# Kernel launches issued through this module since the last reset (bench accounting).
launch_count = 0


def _count(n: int = 1) -> None:
    global launch_count
    launch_count += n


def reset_launch_count() -> int:
    global launch_count
    n = launch_count
    launch_count = 0
    return n


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5, residual: torch.Tensor | None = None,
             out: torch.Tensor | None = None):
    """RMSNorm with optional fused residual add. Returns (normed, residual_stream).

    With `residual`, the residual tensor is updated in place to x + residual and returned as the stream."""
    if not x.is_cuda:
        y, r = reference.rms_norm(x, weight, eps, residual)
        if residual is not None:
            residual.copy_(r.to(residual.dtype))
            return y.to(x.dtype), residual
        return y.to(x.dtype), x
    C = _ext.require()
    if out is None:
        out = torch.empty_like(x)
    C.rmsnorm(x, residual, weight, out, None, None, eps)
    _count()
    return out, (residual if residual is not None else x)


def rms_norm_quant(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5, residual: torch.Tensor | None = None,
                   out_q: torch.Tensor | None = None, out_s: torch.Tensor | None = None):
    """RMSNorm that also emits the row as e4m3 with one f32 scale per 128 columns.
    Returns (normed bf16, q e4m3, scales f32 [rows, H/128], residual_stream). `out_q` / `out_s` (contiguous, CUDA
    only) let the quantised row land where a fused all-gather will pick it up."""
    if not x.is_cuda:
        y, r = reference.rms_norm(x, weight, eps, residual)
        if residual is not None:
            residual.copy_(r.to(residual.dtype))
        yb = y.to(x.dtype)
        q, s = reference.quant_e4m3_1x128(yb.reshape(-1, yb.shape[-1]))
        return yb, q, s, (residual if residual is not None else x)
    C = _ext.require()
    out = torch.empty_like(x)
    rows = x.numel() // x.shape[-1]
    q = out_q if out_q is not None else torch.empty(rows, x.shape[-1], dtype=torch.float8_e4m3fn, device=x.device)
    s = out_s if out_s is not None else torch.empty(rows, x.shape[-1] // 128, dtype=torch.float32, device=x.device)
    C.rmsnorm(x, residual, weight, out, q, s, eps)
    _count()
    return out, q, s, (residual if residual is not None else x)


def quant_e4m3(x: torch.Tensor, out_q: torch.Tensor | None = None, out_s: torch.Tensor | None = None):
    """Per-row 1x128 dynamic e4m3 quantisation of a [M, K] bf16 matrix."""
    if not x.is_cuda:
        return reference.quant_e4m3_1x128(x)
    C = _ext.require()
    q = out_q if out_q is not None else torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
    s = out_s if out_s is not None else torch.empty(x.shape[0], x.shape[1] // 128, dtype=torch.float32, device=x.device)
    C.quant_e4m3(x, q, s)
    _count()
    return q, s


def rope_kvwrite(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor | None, cos_sin: torch.Tensor, positions: torch.Tensor,
                 slots: torch.Tensor | None, k_cache: torch.Tensor | None, v_cache: torch.Tensor | None, head_dim: int,
                 interleaved: bool = False) -> None:
    """Rotate q and k in place ([T, heads*D] views) and scatter k, v into the paged cache."""
    if not q.is_cuda:
        T = q.shape[0]
        qr = reference.apply_rope(q.reshape(T, -1, head_dim), positions, cos_sin, interleaved)
        kr = reference.apply_rope(k.reshape(T, -1, head_dim), positions, cos_sin, interleaved)
        q.copy_(qr.reshape(T, -1).to(q.dtype))
        k.copy_(kr.reshape(T, -1).to(k.dtype))
        if k_cache is not None:
            reference.write_kv(k_cache, v_cache, k.reshape(T, -1, head_dim), v.reshape(T, -1, head_dim), slots)
        return
    C = _ext.require()
    C.rope_kvwrite(q, k, v, cos_sin, positions, slots, k_cache, v_cache, head_dim, interleaved, _state.get(q.device).status)
    _count()


def swiglu(gate_up: torch.Tensor, out: torch.Tensor | None = None, interleaved: bool = False) -> torch.Tensor:
    """silu(gate) * up. Row layout [gate | up], or with `interleaved` alternating blocks of 16 gate and 16 up
    columns (what a plain GEMM against an `interleave_gate_up` weight produces)."""
    if not gate_up.is_cuda:
        if interleaved:
            m = gate_up.shape[0]
            y = gate_up.float().reshape(m, -1, 2, 16)
            return (reference.silu(y[:, :, 0]) * y[:, :, 1]).reshape(m, -1).to(gate_up.dtype)
        return reference.swiglu(gate_up).to(gate_up.dtype)
    C = _ext.require()
    if out is None:
        out = torch.empty(*gate_up.shape[:-1], gate_up.shape[-1] // 2, dtype=gate_up.dtype, device=gate_up.device)
    C.swiglu(gate_up, out, interleaved)
    _count()
    return out


def embedding(ids: torch.Tensor, table: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    if not ids.is_cuda:
        return reference.embedding(ids, table, vocab_start).to(table.dtype)
    C = _ext.require()
    out = torch.empty(ids.numel(), table.shape[1], dtype=table.dtype, device=table.device)
    C.embedding(ids, table, out, vocab_start)
    _count()
    return out


def gather_rows(src: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    if not src.is_cuda:
        return src[index.long()]
    C = _ext.require()
    out = torch.empty(index.numel(), src.shape[1], dtype=src.dtype, device=src.device)
    C.gather_rows(src, index, out, _state.get(src.device).status)
    _count()
    return out


def scatter_rows(src: torch.Tensor, slots: torch.Tensor, dst: torch.Tensor) -> None:
    """dst[slots[i]] = src[i] for slots[i] >= 0 (KV row write for caches with one row per token)."""
    if not src.is_cuda:
        valid = slots >= 0
        dst[slots[valid].long()] = src[valid].to(dst.dtype)
        return
    C = _ext.require()
    C.scatter_rows(src, slots, dst, _state.get(src.device).status)
    _count()


def copy_pages(cache: torch.Tensor, src_pages: torch.Tensor, dst_pages: torch.Tensor) -> None:
    if not cache.is_cuda:
        cache[dst_pages.long()] = cache[src_pages.long()]
        return
    C = _ext.require()
    C.copy_pages(cache, src_pages, dst_pages, _state.get(cache.device).status)
    _count()


PAIR_CONFIG = 1 << 28   # configuration word that selects the CTA-pair (cta_group::2) GEMM kernel; low bits = tile width (256 default, 128)


def _launch_gemm(C, x, w, out, residual, epi, config, st) -> None:
    """One bf16 GEMM launch: the CTA-pair kernel when `config` says so (plain and SwiGLU epilogues only), else the
    single-CTA kernel family with `config` as its tile / split / layout word."""
    if config & PAIR_CONFIG and residual is None and epi != EPI_ADD_RESIDUAL:
        C.gemm_bf16_pair(x, w, out, epi, (config & 0xffff) or 256, st.status)
    else:
        C.gemm_bf16(x, w, out, residual, epi, config & ~PAIR_CONFIG, st.gemm_ws, st.status)


def linear(x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None = None, out: torch.Tensor | None = None,
           config: int = 0) -> torch.Tensor:
    """y = x @ w.T (+ residual) on the tcgen05 GEMM. x [M, K], w [N, K], both bf16."""
    if not x.is_cuda:
        return reference.linear(x, w, residual).to(x.dtype)
    C = _ext.require()
    st = _state.get(x.device)
    if out is None:
        out = torch.empty(x.shape[0], w.shape[0], dtype=x.dtype, device=x.device)
    epi = EPI_ADD_RESIDUAL if residual is not None else EPI_NONE
    if config == 0:
        config = autotune.lookup(x.shape[0], w.shape[0], w.shape[1], epi, x.device.index or 0)
    _launch_gemm(C, x, w, out, residual, epi, config, st)
    _count()
    return out


def linear_pair(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """y = x @ w.T on CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles): the large-M form of `linear`."""
    return linear(x, w, out=out, config=PAIR_CONFIG)


def linear_swiglu(x: torch.Tensor, w_gu: torch.Tensor, out: torch.Tensor | None = None, config: int = 0) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) in one GEMM; `w_gu` is the 16-row interleaved stack from
    `reference.interleave_gate_up`."""
    if not x.is_cuda:
        return reference.linear_swiglu_interleaved(x, w_gu).to(x.dtype)
    C = _ext.require()
    st = _state.get(x.device)
    if out is None:
        out = torch.empty(x.shape[0], w_gu.shape[0] // 2, dtype=x.dtype, device=x.device)
    if config == 0:
        config = autotune.lookup(x.shape[0], w_gu.shape[0], w_gu.shape[1], EPI_SWIGLU, x.device.index or 0)
    _launch_gemm(C, x, w_gu, out, None, EPI_SWIGLU, config, st)
    _count()
    return out


def linear_fp8(x, w_q: torch.Tensor, w_scale: torch.Tensor, out: torch.Tensor | None = None, config: int = 0) -> torch.Tensor:
    """Block-scaled fp8 linear. `x` is either a bf16 [M, K] tensor (quantised here, 1x128 blocks) or a pair
    (x_q e4m3 [M, K], x_scale f32 [M, K/128]) from `rms_norm_quant`. w_q e4m3 [N, K], w_scale f32 [N/128, K/128]."""
    if isinstance(x, tuple):
        xq, xs = x
    else:
        xq, xs = quant_e4m3(x)
    if not xq.is_cuda:
        return reference.linear_fp8_block(xq, xs, w_q, w_scale).to(torch.bfloat16 if w_q.is_cuda else torch.float32)
    C = _ext.require()
    if out is None:
        out = torch.empty(xq.shape[0], w_q.shape[0], dtype=torch.bfloat16, device=xq.device)
    st = _state.get(xq.device)
    C.gemm_fp8(xq, xs, w_q, w_scale, out, config, st.status, st.gemm_ws)   # the workspace enables split-K for under-filled grids
    _count()
    return out


GGML_Q4_K, GGML_Q6_K = 12, 14
_GGML_BLOCK_BYTES = {GGML_Q4_K: 144, GGML_Q6_K: 210}


def gguf_dequant(w_q: torch.Tensor, ggml_type: int, shape) -> torch.Tensor:
    """Packed Q4_K / Q6_K super-blocks (uint8) -> bf16 tensor of `shape` (rows x K, K a multiple of 256)."""
    if not w_q.is_cuda:
        return reference.gguf_dequant(w_q, ggml_type, shape)
    C = _ext.require()
    out = torch.empty(*shape, dtype=torch.bfloat16, device=w_q.device)
    C.gguf_dequant(w_q, ggml_type, out)
    _count()
    return out


def linear_gguf(x: torch.Tensor, w_q: torch.Tensor, ggml_type: int, n_out: int) -> torch.Tensor:
    """y = x @ dequant(w_q).T with the dequantisation fused into the GEMM (decode-sized M); larger M dequantises once
    and runs the bf16 GEMM."""
    K = x.shape[1]
    if not x.is_cuda:
        return reference.linear(x, reference.gguf_dequant(w_q, ggml_type, (n_out, K))).to(x.dtype)
    if x.shape[0] > 128:
        return linear(x, gguf_dequant(w_q, ggml_type, (n_out, K)))
    C = _ext.require()
    y = torch.empty(x.shape[0], n_out, dtype=x.dtype, device=x.device)
    C.gemm_gguf(x, w_q, ggml_type, y, _state.get(x.device).status)
    _count()
    return y


def gemm_config(swap: bool, bn: int, splits: int = 1, stream_k: bool = False) -> int:
    """Encode an explicit GEMM configuration (for tuning sweeps): operand swap, UMMA N, split-K factor, or
    stream-K balancing of the ragged last wave (excludes split-K)."""
    return (int(swap) << 30) | (int(stream_k) << 29) | ((1 if stream_k else splits) << 16) | bn


class AttnMeta:
    """Device-side description of one ragged batch (decode sequences first, then prefill chunks).

    Optional extras, both built on the host by the model runner:
      work, n_items   (sequence, query tile) items of the prefill chunks, longest context first, as an int32 [n, 2] device
                      tensor whose sequence index counts from the first prefill sequence; the tcgen05 prefill kernel then
                      launches exactly one CTA per item and head
      static          a `StaticAttn`: every shape and grid fixed ahead of the batch, so that the launches can sit in a
                      CUDA graph that serves any batch of its bucket
    """

    __slots__ = ("cu_q", "ctx_lens", "block_tables", "num_decode", "num_seqs", "max_q_len", "num_tokens", "max_ctx", "work", "n_items", "static")

    def __init__(self, cu_q, ctx_lens, block_tables, num_decode, max_q_len, max_ctx=0, work=None, n_items=0, static=None):
        self.cu_q, self.ctx_lens, self.block_tables = cu_q, ctx_lens, block_tables
        self.num_decode = int(num_decode)
        self.num_seqs = int(ctx_lens.numel()) if ctx_lens is not None else 0
        self.max_q_len = int(max_q_len)
        self.num_tokens = None
        self.max_ctx = int(max_ctx)
        self.work, self.n_items = work, int(n_items)
        self.static = static


class StaticAttn:
    """Attention metadata of a captured step. The decode launch covers the first `d_rows` token rows: row i < number of
    decode sequences has its context length in `d_ctx[i]`, every other row has 0 there (the kernel writes zeros, which
    the prefill launch then overwrites where the row belongs to a chunk). The prefill launch covers `max_items` work
    items of which the first `n_work[0]` are valid; `p_cu` / `p_ctx` / `p_bt` describe the prefill sequences only
    (`p_cu` holds absolute token rows; unused entries repeat the last offset)."""

    __slots__ = ("d_rows", "d_ctx", "d_bt", "d_splits", "p_cu", "p_ctx", "p_bt", "work", "n_work", "max_items", "max_q_len")

    def __init__(self, d_rows, d_ctx, d_bt, d_splits, p_cu, p_ctx, p_bt, work, n_work, max_items, max_q_len):
        self.d_rows, self.d_ctx, self.d_bt, self.d_splits = int(d_rows), d_ctx, d_bt, int(d_splits)
        self.p_cu, self.p_ctx, self.p_bt = p_cu, p_ctx, p_bt
        self.work, self.n_work, self.max_items, self.max_q_len = work, n_work, int(max_items), int(max_q_len)


def prefill_work_items(cu_q, ctx_lens, num_decode: int, tile: int = 128):
    """Host-side work list of the prefill chunks of one batch: an int32 [n, 2] numpy array of (prefill sequence index,
    query tile), ordered by the number of KV tiles each item visits, longest first (the CTAs that take longest start
    first). `cu_q` [B + 1] and `ctx_lens` [B] are the batch's host arrays."""
    import numpy as np

    cu = np.asarray(cu_q[num_decode:], dtype=np.int64)
    ctx = np.asarray(ctx_lens[num_decode:], dtype=np.int64)
    q_len = cu[1:] - cu[:-1]
    tiles = (q_len + tile - 1) // tile
    n = int(tiles.sum())
    if n == 0:
        return np.zeros((0, 2), dtype=np.int32)
    seq = np.repeat(np.arange(len(tiles), dtype=np.int64), tiles)
    first = np.cumsum(tiles) - tiles
    qt = np.arange(n, dtype=np.int64) - np.repeat(first, tiles)
    rows = np.minimum(tile, q_len[seq] - qt * tile)
    kv_tiles = np.minimum((ctx[seq] - q_len[seq] + qt * tile + rows + tile - 1) // tile, (ctx[seq] + tile - 1) // tile)
    order = np.argsort(-kv_tiles, kind="stable")
    return np.stack([seq[order], qt[order]], axis=1).astype(np.int32)


def _decode_splits(batch: int, n_kv: int, max_ctx: int) -> int:
    """Split the KV range so that small batches still fill the machine: the decode kernel runs one warp per
    (split, kv head, sequence) with four such CTAs per SM (148 SMs x 4 = 592 per wave)."""
    ctas = batch * n_kv
    if ctas >= 1184 or max_ctx <= 256:
        return 1
    want = (1184 + ctas - 1) // ctas
    return max(1, min(want, max_ctx // 128, 32))


def _decode_launches(splits: int, page_size: int) -> int:
    """Kernels one decode-attention call launches: the split that finishes last merges the partials itself on the TMA
    path (page sizes that are multiples of 32); the cp.async path merges with a second kernel."""
    return 1 if splits == 1 or page_size % 32 == 0 else 2


# Prefill attention on tcgen05 for head_dim 128 and 128-token pages (False: the mma.sync kernel for every shape).
prefill_tensor_core = True


def prefill_on_tensor_core(head_dim: int, page_size: int) -> bool:
    return bool(prefill_tensor_core and head_dim == 128 and page_size == 128)


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, meta: AttnMeta, scale: float,
                    head_dim: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """Causal GQA attention over the paged cache. q, out: [T, n_q * D]."""
    if not q.is_cuda:
        T = q.shape[0]
        o = reference.paged_attention(q.reshape(T, -1, head_dim), k_cache, v_cache, meta.cu_q, meta.ctx_lens,
                                      meta.block_tables, scale)
        return o.reshape(T, -1).to(q.dtype)
    C = _ext.require()
    st = _state.get(q.device)
    if out is None:
        out = torch.empty(q.shape[0], q.shape[1], dtype=q.dtype, device=q.device)
    sa = meta.static
    if sa is not None:
        # captured step: fixed grids, everything that varies is read from device memory
        if sa.d_rows > 0:
            C.attn_decode(q[:sa.d_rows], k_cache, v_cache, out[:sa.d_rows], sa.d_ctx, sa.d_bt, st.attn_ws, head_dim, sa.d_splits,
                          scale, st.status, st.attn_counters)
            _count(_decode_launches(sa.d_splits, k_cache.shape[2]))
        if sa.max_items > 0:
            C.attn_prefill_tc(q, k_cache, v_cache, out, sa.p_cu, sa.p_ctx, sa.p_bt, sa.max_q_len, scale, 0, st.status,
                              sa.work, sa.n_work, sa.max_items)
            _count()
        return out
    nd, ns = meta.num_decode, meta.num_seqs
    if nd > 0:
        splits = _decode_splits(nd, k_cache.shape[1], meta.max_ctx)
        C.attn_decode(q[:nd], k_cache, v_cache, out[:nd], meta.ctx_lens[:nd], meta.block_tables[:nd], st.attn_ws, head_dim,
                      splits, scale, st.status, st.attn_counters)
        _count(_decode_launches(splits, k_cache.shape[2]))
    if ns > nd:
        # cu_q offsets are absolute token rows, so q/out are passed whole
        if prefill_on_tensor_core(head_dim, k_cache.shape[2]):
            # tcgen05 / TMEM kernel: one KV tile = one 128-token page
            if meta.work is not None and meta.n_items > 0:
                C.attn_prefill_tc(q, k_cache, v_cache, out, meta.cu_q[nd:], meta.ctx_lens[nd:], meta.block_tables[nd:],
                                  meta.max_q_len, scale, 0, st.status, meta.work, None, meta.n_items)
            else:
                C.attn_prefill_tc(q, k_cache, v_cache, out, meta.cu_q[nd:], meta.ctx_lens[nd:], meta.block_tables[nd:],
                                  meta.max_q_len, scale, 0, st.status)
        else:
            C.attn_prefill(q, k_cache, v_cache, out, meta.cu_q[nd:], meta.ctx_lens[nd:], meta.block_tables[nd:], head_dim,
                           meta.max_q_len, scale, st.status)
        _count()
    return out


def mla_decode(q_lat: torch.Tensor, q_rope: torch.Tensor, kv_cache: torch.Tensor, ctx_lens: torch.Tensor,
               block_tables: torch.Tensor, scale: float, max_ctx: int = 0) -> torch.Tensor:
    """Absorbed multi-head latent attention for one query token per sequence.
    q_lat [B, H, 512], q_rope [B, H, 64], kv_cache [pages, page_size, 576] -> attention output in latent space [B, H, 512]."""
    if not q_lat.is_cuda:
        return reference.mla_decode(q_lat, q_rope, kv_cache, ctx_lens, block_tables, scale).to(q_lat.dtype)
    C = _ext.require()
    st = _state.get(q_lat.device)
    B, H = q_lat.shape[0], q_lat.shape[1]
    ctas = B * ((H + 15) // 16)
    splits = 1
    if ctas < 148 and max_ctx > 256:
        splits = max(1, min((148 + ctas - 1) // ctas, max_ctx // 128, 16))
    out = torch.empty_like(q_lat)
    C.mla_decode(q_lat, q_rope, kv_cache, out, ctx_lens, block_tables, st.attn_ws, splits, scale, st.status)
    _count(2 if splits > 1 else 1)
    return out


def mla_attend(q_lat: torch.Tensor, q_rope: torch.Tensor, kv_cache: torch.Tensor, meta: "AttnMeta", scale: float) -> torch.Tensor:
    """Absorbed multi-head latent attention over a whole engine batch in one launch: decode tokens and the tokens of
    prefill chunks alike (the chunk's latents must already be in the cache). q_lat [T, H, 512] and q_rope [T, H, 64]
    may be column slices of one projection output (strided rows). Returns [T, H, 512] in latent space."""
    if not q_lat.is_cuda:
        return reference.mla_attend(q_lat, q_rope, kv_cache, meta.cu_q, meta.ctx_lens, meta.block_tables, scale).to(q_lat.dtype)
    C = _ext.require()
    st = _state.get(q_lat.device)
    T, H = q_lat.shape[0], q_lat.shape[1]
    out = torch.empty(T, H, 512, dtype=q_lat.dtype, device=q_lat.device)
    if T == 0:
        return out
    decode_only = meta.num_decode == meta.num_seqs
    if decode_only:
        row_ctx, row_seq = meta.ctx_lens, None      # one row per sequence, in order
        n_meta = 0
    else:
        row_ctx = torch.empty(T, dtype=torch.int32, device=q_lat.device)
        row_seq = torch.empty(T, dtype=torch.int32, device=q_lat.device)
        C.mla_rows_meta(meta.cu_q, meta.ctx_lens, row_ctx, row_seq)
        n_meta = 1
    ctas = T * ((H + 15) // 16)
    splits = 1
    if ctas < 148 and meta.max_ctx > 256:
        splits = max(1, min((148 + ctas - 1) // ctas, meta.max_ctx // 128, 16))
    C.mla_attend(q_lat, q_rope, kv_cache, out, row_ctx, meta.block_tables, row_seq, st.attn_ws, splits, scale, st.status)
    _count(n_meta + (2 if splits > 1 else 1))
    return out


def argmax(logits: torch.Tensor) -> torch.Tensor:
    if not logits.is_cuda:
        return torch.argmax(logits.float(), dim=-1)
    C = _ext.require()
    ids = torch.empty(logits.shape[0], dtype=torch.int64, device=logits.device)
    C.argmax(logits, ids, None)
    _count()
    return ids


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor, seed: int, step: int,
           uniforms: torch.Tensor | None = None) -> torch.Tensor:
    """Per-row temperature / top-k / top-p sampling. temperature == 0 selects greedy for that row."""
    if not logits.is_cuda:
        ids = []
        for r in range(logits.shape[0]):
            u = float(uniforms[r]) if uniforms is not None else reference.philox_uniform(seed, step, r)
            ids.append(reference.sample(logits[r], float(temperature[r]), int(top_k[r]), float(top_p[r]), u))
        return torch.tensor(ids, dtype=torch.int64)
    C = _ext.require()
    ids = torch.empty(logits.shape[0], dtype=torch.int64, device=logits.device)
    C.sample(logits, ids, temperature, top_k, top_p, uniforms, seed, step)
    _count()
    return ids
