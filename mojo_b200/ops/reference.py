"""Plain PyTorch fp32 reference implementation of every op in `mojo_b200.ops`.

This is the oracle the CUDA kernels are tested against and the compute path of the CPU engine. It mirrors the
reference project's testing idea of a scalar oracle per vectorised function (`libm_call`,
stdlib/test/test_utils/test_utils.mojo:19-44): simple, obviously-correct code in full precision. Inputs of any
float dtype are upcast to fp32; outputs are returned in fp32 unless stated otherwise.
"""
from __future__ import annotations

import math

import torch

# ------------------------------------------------------------------------------------------------------
# normalisation / activation / embedding
# ------------------------------------------------------------------------------------------------------


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5, residual: torch.Tensor | None = None):
    """Returns (normed, new_residual). new_residual = x + residual (or x when residual is None)."""
    xf = x.float()
    if residual is not None:
        xf = xf + residual.float()
        # the residual stream is stored in the activation dtype; normalise the stored value
        xf = xf.to(x.dtype).float()
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    y = xf * torch.rsqrt(var + eps) * weight.float()
    return y, xf


def silu(x: torch.Tensor) -> torch.Tensor:
    xf = x.float()
    return xf * torch.sigmoid(xf)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    f = gate_up.shape[-1] // 2
    return silu(gate_up[..., :f]) * gate_up[..., f:].float()


def embedding(ids: torch.Tensor, table: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    local = ids - vocab_start
    inside = (local >= 0) & (local < table.shape[0])
    out = table.float()[local.clamp(0, table.shape[0] - 1)]
    return out * inside.unsqueeze(-1)


# ------------------------------------------------------------------------------------------------------
# rotary embedding
# ------------------------------------------------------------------------------------------------------


def rope_inv_freq(rot_dim: int, theta: float, scaling: dict | None = None) -> torch.Tensor:
    """Inverse frequencies in float64; `scaling` implements the Llama-3.1 'llama3' frequency rescale."""
    inv = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float64) / rot_dim))
    if scaling and scaling.get("rope_type", scaling.get("type")) == "llama3":
        factor = float(scaling["factor"])
        low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
        old = float(scaling["original_max_position_embeddings"])
        wavelen = 2 * math.pi / inv
        smooth = ((old / wavelen) - low) / (high - low)
        scaled = torch.where(wavelen > old / low, inv / factor, inv)
        mid = (wavelen <= old / low) & (wavelen >= old / high)
        scaled = torch.where(mid, (1 - smooth) * inv / factor + smooth * inv, scaled)
        inv = scaled
    return inv


def rope_table(max_pos: int, rot_dim: int, theta: float, scaling: dict | None = None) -> torch.Tensor:
    """f32 [max_pos, rot_dim]: cos in the first half of a row, sin in the second half."""
    inv = rope_inv_freq(rot_dim, theta, scaling)
    ang = torch.arange(max_pos, dtype=torch.float64).unsqueeze(1) * inv.unsqueeze(0)
    return torch.cat([ang.cos(), ang.sin()], dim=1).float()


def apply_rope(x: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor, interleaved: bool = False) -> torch.Tensor:
    """x: [T, heads, D]; rotates the first rot_dim = cos_sin.shape[1] elements of every head."""
    rot = cos_sin.shape[1]
    half = rot // 2
    cs = cos_sin[positions.long()]
    cos, sin = cs[:, None, :half].float(), cs[:, None, half:].float()
    xf = x.float().clone()
    xr = xf[..., :rot]
    if interleaved:
        a, b = xr[..., 0::2], xr[..., 1::2]
        out = torch.stack([a * cos - b * sin, b * cos + a * sin], dim=-1).flatten(-2)
    else:
        a, b = xr[..., :half], xr[..., half:]
        out = torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)
    xf[..., :rot] = out
    return xf


# ------------------------------------------------------------------------------------------------------
# paged attention
# ------------------------------------------------------------------------------------------------------


def write_kv(k_cache: torch.Tensor, v_cache: torch.Tensor, k: torch.Tensor, v: torch.Tensor, slots: torch.Tensor) -> None:
    """Caches are [pages, n_kv, page_size, D]; k, v are [T, n_kv, D]; slot = page * page_size + offset."""
    page_size = k_cache.shape[2]
    valid = slots >= 0
    s = slots[valid].long()
    page, off = s // page_size, s % page_size
    k_cache[page, :, off] = k[valid].to(k_cache.dtype)
    v_cache[page, :, off] = v[valid].to(v_cache.dtype)


def gather_kv(cache: torch.Tensor, block_table: torch.Tensor, ctx_len: int) -> torch.Tensor:
    """[ctx_len, n_kv, D] view of one sequence's cache contents."""
    page_size = cache.shape[2]
    n_pages = (ctx_len + page_size - 1) // page_size
    pages = cache[block_table[:n_pages].long()]  # [n_pages, n_kv, page_size, D]
    return pages.permute(0, 2, 1, 3).reshape(n_pages * page_size, cache.shape[1], cache.shape[3])[:ctx_len]


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, cu_q: torch.Tensor, ctx_lens: torch.Tensor,
                    block_tables: torch.Tensor, scale: float) -> torch.Tensor:
    """Causal GQA attention for a ragged batch of query chunks. q: [T, n_q, D] -> [T, n_q, D] fp32.

    Sequence b owns query rows cu_q[b]:cu_q[b+1]; these are the last q_len positions of a context of ctx_lens[b]
    tokens whose keys/values are all in the cache already.
    """
    T, n_q, D = q.shape
    n_kv = k_cache.shape[1]
    group = n_q // n_kv
    out = torch.zeros(T, n_q, D, dtype=torch.float32, device=q.device)
    for b in range(ctx_lens.numel()):
        s, e = int(cu_q[b]), int(cu_q[b + 1])
        ql, ctx = e - s, int(ctx_lens[b])
        if ql == 0:
            continue
        k = gather_kv(k_cache, block_tables[b], ctx).float()  # [ctx, n_kv, D]
        v = gather_kv(v_cache, block_tables[b], ctx).float()
        k = k.repeat_interleave(group, dim=1)
        v = v.repeat_interleave(group, dim=1)
        qq = q[s:e].float()  # [ql, n_q, D]
        scores = torch.einsum("qhd,khd->hqk", qq, k) * scale
        qpos = torch.arange(ctx - ql, ctx, device=q.device).unsqueeze(1)
        kpos = torch.arange(ctx, device=q.device).unsqueeze(0)
        scores = scores.masked_fill(~(kpos <= qpos).unsqueeze(0), float("-inf"))
        p = torch.softmax(scores, dim=-1)
        out[s:e] = torch.einsum("hqk,khd->qhd", p, v)
    return out


# ------------------------------------------------------------------------------------------------------
# GEMM and quantisation
# ------------------------------------------------------------------------------------------------------


def linear(x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
    """y = x @ w.T (+ residual) in fp32. w is [N, K] like nn.Linear.weight."""
    y = x.float() @ w.float().t()
    if residual is not None:
        y = y + residual.float()
    return y


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor, block: int = 16) -> torch.Tensor:
    """Stack gate and up projection rows in alternating blocks of `block` rows:
    rows [32b, 32b+16) = gate rows [16b, 16b+16), rows [32b+16, 32b+32) = up rows [16b, 16b+16).
    This is the weight layout the SwiGLU GEMM epilogue expects."""
    f, k = w_gate.shape
    assert f % block == 0 and w_up.shape == w_gate.shape
    g = w_gate.reshape(f // block, block, k)
    u = w_up.reshape(f // block, block, k)
    return torch.stack([g, u], dim=1).reshape(2 * f, k).contiguous()


def deinterleave_gate_up(w_gu: torch.Tensor, block: int = 16):
    """Inverse of `interleave_gate_up`: (w_gate [F, K], w_up [F, K])."""
    two_f, k = w_gu.shape
    v = w_gu.reshape(two_f // (2 * block), 2, block, k)
    return v[:, 0].reshape(two_f // 2, k).contiguous(), v[:, 1].reshape(two_f // 2, k).contiguous()


def linear_swiglu_interleaved(x: torch.Tensor, w_gu: torch.Tensor, block: int = 16) -> torch.Tensor:
    """silu(x @ Wg.T) * (x @ Wu.T) for a weight stored by `interleave_gate_up`."""
    y = x.float() @ w_gu.float().t()  # [M, 2F] interleaved
    m = y.shape[0]
    y = y.reshape(m, -1, 2, block)
    return (silu(y[:, :, 0]) * y[:, :, 1]).reshape(m, -1)


E4M3_MAX = 448.0


def quant_e4m3_1x128(x: torch.Tensor):
    """Per-row, per-128-column dynamic quantisation: returns (q float8_e4m3fn [M, K], scale f32 [M, K/128])."""
    m, k = x.shape
    xf = x.float().reshape(m, k // 128, 128)
    amax = xf.abs().amax(dim=-1).clamp_min(1e-10)
    scale = amax / E4M3_MAX
    q = (xf / scale.unsqueeze(-1)).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.reshape(m, k), scale


def quant_e4m3_128x128(w: torch.Tensor):
    """Weight quantisation with one scale per 128x128 block: (q [N, K] e4m3, scale f32 [ceil(N/128), ceil(K/128)])."""
    n, k = w.shape
    nb, kb = (n + 127) // 128, (k + 127) // 128
    wp = torch.zeros(nb * 128, kb * 128, dtype=torch.float32, device=w.device)
    wp[:n, :k] = w.float()
    blocks = wp.reshape(nb, 128, kb, 128)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-10)
    scale = amax / E4M3_MAX
    q = (blocks / scale[:, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).reshape(nb * 128, kb * 128)[:n, :k]
    return q.to(torch.float8_e4m3fn).contiguous(), scale


def dequant_e4m3_128x128(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    n, k = q.shape
    s = scale.repeat_interleave(128, dim=0)[:n].repeat_interleave(128, dim=1)[:, :k]
    return q.float() * s


def linear_fp8_block(xq: torch.Tensor, xs: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor) -> torch.Tensor:
    """Block-scaled fp8 GEMM oracle: dequantise both operands to fp32 and multiply."""
    x = xq.float() * xs.repeat_interleave(128, dim=1)[:, : xq.shape[1]]
    w = dequant_e4m3_128x128(wq, ws)
    return x @ w.t()


# ------------------------------------------------------------------------------------------------------
# sampling
# ------------------------------------------------------------------------------------------------------

_PHILOX_M0, _PHILOX_M1 = 0xD2511F53, 0xCD9E8D57
_PHILOX_W0, _PHILOX_W1 = 0x9E3779B9, 0xBB67AE85


def philox_uniform(seed: int, step: int, row: int) -> float:
    """Philox4x32-10 with counter (step_lo, step_hi, row, 0) and key (seed_lo, seed_hi); returns the first
    output word mapped to [0, 1) with 24 bits. Must match the device generator bit for bit."""
    c = [step & 0xFFFFFFFF, (step >> 32) & 0xFFFFFFFF, row & 0xFFFFFFFF, 0]
    k = [seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF]
    for i in range(10):
        p0 = _PHILOX_M0 * c[0]
        p1 = _PHILOX_M1 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & 0xFFFFFFFF, p1 & 0xFFFFFFFF, ((p0 >> 32) ^ c[3] ^ k[1]) & 0xFFFFFFFF, p0 & 0xFFFFFFFF]
        if i < 9:
            k = [(k[0] + _PHILOX_W0) & 0xFFFFFFFF, (k[1] + _PHILOX_W1) & 0xFFFFFFFF]
    return (c[0] >> 8) / 16777216.0


def sample_keep_mask(logits: torch.Tensor, temperature: float, top_k: int, top_p: float) -> torch.Tensor:
    """Boolean mask of tokens that survive top-k then top-p (ties at a threshold are all kept)."""
    x = logits.float()
    v = x.numel()
    keep = torch.ones(v, dtype=torch.bool, device=x.device)
    if 0 < top_k < v:
        kth = torch.topk(x, top_k).values[-1]
        keep &= x >= kth
    if top_p < 1.0:
        w = torch.where(keep, torch.exp((x - x.max()) / temperature), torch.zeros_like(x)).double()
        z = w.sum()
        order = torch.argsort(x, descending=True, stable=True)
        cum_before = torch.cumsum(w[order], 0) - w[order]
        # smallest set of largest values whose mass reaches top_p * z; equal values share a fate
        inside_sorted = cum_before < top_p * z
        thr = x[order][inside_sorted].min()
        keep &= x >= thr
    return keep


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, u: float) -> int:
    """Inverse-CDF draw in index order over the kept set, for one row."""
    x = logits.float()
    if temperature <= 0.0:
        return int(torch.argmax(x))
    keep = sample_keep_mask(x, temperature, top_k, top_p)
    w = torch.where(keep, torch.exp((x - x.max()) / temperature), torch.zeros_like(x)).double()
    cdf = torch.cumsum(w, 0)
    target = u * float(cdf[-1])
    idx = int(torch.searchsorted(cdf, torch.tensor(target, dtype=torch.float64), right=True))
    return min(idx, x.numel() - 1)


# ------------------------------------------------------------------------------------------------------
# MLA (multi-head latent attention), absorbed form
# ------------------------------------------------------------------------------------------------------


def mla_decode(q_lat: torch.Tensor, q_rope: torch.Tensor, kv_cache: torch.Tensor, ctx_lens: torch.Tensor,
               block_tables: torch.Tensor, scale: float) -> torch.Tensor:
    """q_lat [B, H, R], q_rope [B, H, P]; kv_cache [pages, page_size, R + P] (latent then rope key).
    Returns the attention output in latent space [B, H, R] (to be multiplied by W_UV by the caller)."""
    B, H, R = q_lat.shape
    page_size = kv_cache.shape[1]
    out = torch.zeros(B, H, R, dtype=torch.float32, device=q_lat.device)
    for b in range(B):
        ctx = int(ctx_lens[b])
        n_pages = (ctx + page_size - 1) // page_size
        kv = kv_cache[block_tables[b, :n_pages].long()].reshape(n_pages * page_size, -1)[:ctx].float()
        lat, rope = kv[:, :R], kv[:, R:]
        s = (q_lat[b].float() @ lat.t() + q_rope[b].float() @ rope.t()) * scale
        p = torch.softmax(s, dim=-1)
        out[b] = p @ lat
    return out


def mla_attend(q_lat: torch.Tensor, q_rope: torch.Tensor, kv_cache: torch.Tensor, cu_q: torch.Tensor, ctx_lens: torch.Tensor,
               block_tables: torch.Tensor, scale: float) -> torch.Tensor:
    """Absorbed latent attention for a mixed batch: q_lat [T, H, R], q_rope [T, H, P] hold the query tokens of every
    sequence back to back (`cu_q` offsets); token i of a chunk of q_len tokens sees the first ctx - q_len + i + 1 cache
    positions of its sequence. Returns [T, H, R] in latent space."""
    T, H, R = q_lat.shape
    page_size = kv_cache.shape[1]
    out = torch.zeros(T, H, R, dtype=torch.float32, device=q_lat.device)
    cu = [int(v) for v in cu_q]
    for b in range(len(cu) - 1):
        s0, e0, ctx = cu[b], cu[b + 1], int(ctx_lens[b])
        if e0 == s0 or ctx == 0:
            continue
        n_pages = (ctx + page_size - 1) // page_size
        kv = kv_cache[block_tables[b, :n_pages].long()].reshape(n_pages * page_size, -1)[:ctx].float()
        lat, rope = kv[:, :R], kv[:, R:]
        s = (torch.einsum("qhr,kr->hqk", q_lat[s0:e0].float(), lat) + torch.einsum("qhp,kp->hqk", q_rope[s0:e0].float(), rope)) * scale
        qpos = torch.arange(ctx - (e0 - s0), ctx, device=s.device).unsqueeze(1)
        kpos = torch.arange(ctx, device=s.device).unsqueeze(0)
        s = s.masked_fill(~(kpos <= qpos).unsqueeze(0), float("-inf"))
        out[s0:e0] = torch.einsum("hqk,kr->qhr", torch.softmax(s, dim=-1), lat)
    return out


# ------------------------------------------------------------------------------------------------------
# MoE
# ------------------------------------------------------------------------------------------------------


def moe_route(router_logits: torch.Tensor, top_k: int, norm_topk: bool = False, scale: float = 1.0):
    """Softmax over all experts, then top-k (DeepSeek-V2 'greedy' routing). Returns (weights [T, k], ids [T, k])."""
    p = torch.softmax(router_logits.float(), dim=-1)
    w, idx = torch.topk(p, top_k, dim=-1)
    if norm_topk:
        w = w / w.sum(dim=-1, keepdim=True)
    return w * scale, idx


def moe_forward(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, weights: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """x [T, H]; w_gate_up [E, 2F, H] (gate rows then up rows); w_down [E, H, F]. Dense loop over experts."""
    T, H = x.shape
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    xf = x.float()
    for e in range(w_gate_up.shape[0]):
        tok, slot = torch.where(ids == e)
        if tok.numel() == 0:
            continue
        h = swiglu(xf[tok] @ w_gate_up[e].float().t())
        y = h @ w_down[e].float().t()
        out.index_add_(0, tok, y * weights[tok, slot].unsqueeze(-1).float())
    return out


# ------------------------------------------------------------------------------------------------------
# GGUF k-quants
# ------------------------------------------------------------------------------------------------------


def gguf_dequant(w_q: torch.Tensor, ggml_type: int, shape) -> torch.Tensor:
    """Q4_K (type 12) / Q6_K (type 14) super-blocks -> fp32, restated from the block layout (256 weights per block:
    Q4_K = f16 d, f16 dmin, 12 packed 6-bit scales/mins, 128 nibble bytes; Q6_K = 128 low-nibble bytes, 64 bytes of
    2-bit highs, 16 int8 scales, f16 d)."""
    import numpy as np

    raw = w_q.detach().cpu().numpy().view(np.uint8).reshape(-1)
    if ggml_type == 12:
        b = raw.reshape(-1, 144)
        d = b[:, 0:2].copy().view(np.float16).astype(np.float32)
        dmin = b[:, 2:4].copy().view(np.float16).astype(np.float32)
        sc = b[:, 4:16].astype(np.int32)
        qs = b[:, 16:144]
        scales = np.zeros((b.shape[0], 8), np.float32)
        mins = np.zeros((b.shape[0], 8), np.float32)
        for j in range(8):
            if j < 4:
                scales[:, j] = sc[:, j] & 63
                mins[:, j] = sc[:, j + 4] & 63
            else:
                scales[:, j] = (sc[:, j + 4] & 0xF) | ((sc[:, j - 4] >> 6) << 4)
                mins[:, j] = (sc[:, j + 4] >> 4) | ((sc[:, j] >> 6) << 4)
        out = np.zeros((b.shape[0], 256), np.float32)
        for j in range(8):
            q = qs[:, (j // 2) * 32:(j // 2) * 32 + 32]
            q = (q >> 4) if (j & 1) else (q & 0xF)
            out[:, j * 32:(j + 1) * 32] = d * scales[:, j:j + 1] * q - dmin * mins[:, j:j + 1]
    elif ggml_type == 14:
        b = raw.reshape(-1, 210)
        ql, qh = b[:, :128].astype(np.int32), b[:, 128:192].astype(np.int32)
        sc = b[:, 192:208].copy().view(np.int8).astype(np.float32)
        d = b[:, 208:210].copy().view(np.float16).astype(np.float32)
        out = np.zeros((b.shape[0], 256), np.float32)
        for half in range(2):
            for quarter in range(4):
                l = np.arange(32)
                lo = ql[:, half * 64 + (quarter & 1) * 32 + l]
                lo = (lo >> 4) if quarter >= 2 else (lo & 0xF)
                hi = (qh[:, half * 32 + l] >> (2 * quarter)) & 3
                q = (lo | (hi << 4)) - 32
                s_ = sc[:, half * 8 + quarter * 2 + (l >> 4)]
                out[:, half * 128 + quarter * 32:half * 128 + quarter * 32 + 32] = d * s_ * q
    else:
        raise ValueError(f"unsupported ggml type {ggml_type}")
    return torch.from_numpy(out.reshape(shape))


def random_gguf_blocks(n_blocks: int, ggml_type: int, seed: int = 0) -> torch.Tensor:
    """Random but well-formed super-blocks (finite f16 scales) for tests."""
    import numpy as np

    rng = np.random.default_rng(seed)
    nb = 144 if ggml_type == 12 else 210
    b = rng.integers(0, 256, size=(n_blocks, nb), dtype=np.uint8)
    if ggml_type == 12:
        b[:, 0:2] = rng.uniform(0.001, 0.02, size=(n_blocks, 1)).astype(np.float16).view(np.uint8)
        b[:, 2:4] = rng.uniform(0.001, 0.02, size=(n_blocks, 1)).astype(np.float16).view(np.uint8)
    else:
        b[:, 208:210] = rng.uniform(0.0005, 0.004, size=(n_blocks, 1)).astype(np.float16).view(np.uint8)
    return torch.from_numpy(b.reshape(-1))
