// Memory-bound kernels: RMSNorm (+residual, +fp8 activation quant), RoPE + paged KV write, SwiGLU,
// embedding / row gathers, KV page copies. All math in f32 (half types accumulate in f32, the rule of
// stdlib/src/utils/numerics.mojo:1031-1054); rsqrt/rcp/ex2 are the `.approx.ftz` forms the reference
// picks on NVIDIA targets (stdlib/src/math/math.mojo:263-346, 373-401).
#include <cstdint>
#include <cuda_bf16.h>
#include "b2/api.h"
#include "b2/launch.h"
#include "b2/ptx.cuh"
#include "b2/vec.cuh"

namespace b2 {
namespace {

// ------------------------------------------------------------------------------------------------
// RMSNorm: one CTA per row, the row lives in registers (VPT 16-byte vectors per thread).
// ------------------------------------------------------------------------------------------------
template <int VPT, bool QUANT>
__global__ void rmsnorm_kernel(const uint4* __restrict__ x, uint4* __restrict__ residual,
                               const uint4* __restrict__ weight, uint4* __restrict__ out,
                               uint8_t* __restrict__ q_out, float* __restrict__ q_scale, int hidden, float eps) {
  ptx::grid_dep_sync();
  __shared__ float scratch[33];
  const int row = blockIdx.x;
  const int nvec = hidden >> 3;
  const size_t base = static_cast<size_t>(row) * nvec;
  float v[VPT][8];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < nvec) {
      uint4 raw = x[base + c];
      bf16x8_to_f32(raw, v[i]);
      if (residual != nullptr) {
        float r[8];
        bf16x8_to_f32(residual[base + c], r);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] += r[j];
        // The residual stream is stored in bf16; normalise the value that is actually stored.
        uint4 packed = f32_to_bf16x8(v[i]);
        residual[base + c] = packed;
        bf16x8_to_f32(packed, v[i]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = 0.0f;
    }
  }
  ss = block_sum(ss, scratch);
  const float rstd = ptx::rsqrt(ss / static_cast<float>(hidden) + eps);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < nvec) {
      float w[8];
      bf16x8_to_f32(weight[c], w);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = v[i][j] * rstd * w[j];
      uint4 packed = f32_to_bf16x8(v[i]);
      out[base + c] = packed;
      if (QUANT) bf16x8_to_f32(packed, v[i]);  // quantise what the bf16 consumer would have seen
    }
  }
  if (QUANT) {
    // One scale per 128 columns = 16 vectors = 16 consecutive threads (blockDim is a multiple of 32).
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      float amax = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[i][j]));
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      if (c < nvec) {
        const float scale = fmaxf(amax, 1e-10f) * (1.0f / 448.0f);
        const float inv = 1.0f / scale;
        uint2 q;
        q.x = ptx::pack_e4m3x2(v[i][0] * inv, v[i][1] * inv) | (uint32_t(ptx::pack_e4m3x2(v[i][2] * inv, v[i][3] * inv)) << 16);
        q.y = ptx::pack_e4m3x2(v[i][4] * inv, v[i][5] * inv) | (uint32_t(ptx::pack_e4m3x2(v[i][6] * inv, v[i][7] * inv)) << 16);
        reinterpret_cast<uint2*>(q_out + static_cast<size_t>(row) * hidden)[c] = q;
        if ((c & 15) == 0) q_scale[static_cast<size_t>(row) * (hidden >> 7) + (c >> 4)] = scale;
      }
    }
  }
}

__global__ void quant_e4m3_1x128_kernel(const uint4* __restrict__ x, uint8_t* __restrict__ q_out,
                                        float* __restrict__ scale_out, int rows, int cols) {
  ptx::grid_dep_sync();
  // One half-warp (16 lanes x 8 elements) per 128-column group.
  const int groups_per_row = cols >> 7;
  const int64_t gid = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4;
  const int sub = threadIdx.x & 15;
  const int64_t total = static_cast<int64_t>(rows) * groups_per_row;
  const bool active = gid < total;
  float v[8];
  float amax = 0.0f;
  size_t vec_index = 0;
  if (active) {
    const int64_t row = gid / groups_per_row;
    const int g = static_cast<int>(gid % groups_per_row);
    vec_index = static_cast<size_t>(row) * (cols >> 3) + g * 16 + sub;
    bf16x8_to_f32(x[vec_index], v);
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
  }
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (active) {
    const float scale = fmaxf(amax, 1e-10f) * (1.0f / 448.0f);
    const float inv = 1.0f / scale;
    uint2 q;
    q.x = ptx::pack_e4m3x2(v[0] * inv, v[1] * inv) | (uint32_t(ptx::pack_e4m3x2(v[2] * inv, v[3] * inv)) << 16);
    q.y = ptx::pack_e4m3x2(v[4] * inv, v[5] * inv) | (uint32_t(ptx::pack_e4m3x2(v[6] * inv, v[7] * inv)) << 16);
    reinterpret_cast<uint2*>(q_out)[vec_index] = q;
    if (sub == 0) scale_out[gid] = scale;
  }
}

// ------------------------------------------------------------------------------------------------
// RoPE + KV cache scatter. One CTA per token; threads sweep (head, 8-element vector) work items.
// Half-split ("neox") layout pairs element j with j + rot/2; interleaved pairs (2j, 2j+1).
// ------------------------------------------------------------------------------------------------
__global__ void rope_kvwrite_kernel(__nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k,
                                    const __nv_bfloat16* __restrict__ v, const float* __restrict__ cos_sin,
                                    const int32_t* __restrict__ positions, const int64_t* __restrict__ slots,
                                    __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int n_q,
                                    int n_kv, int head_dim, int rot_dim, int interleaved, int64_t q_stride,
                                    int64_t k_stride, int64_t v_stride, int page_size, int64_t num_slots, int max_pos,
                                    Status* status) {
  ptx::grid_dep_sync();
  const int t = blockIdx.x;
  int pos = positions[t];
  if (!B2_ASSERT(status, pos >= 0 && pos < max_pos, kSiteKvIndex, pos, max_pos)) pos = 0;
  const int64_t slot = slots != nullptr ? slots[t] : -1;
  const bool write_cache = slot >= 0 && k_cache != nullptr;
  if (write_cache && !B2_ASSERT(status, slot < num_slots, kSiteKvIndex, slot, num_slots)) return;
  const float* cs = cos_sin + static_cast<size_t>(pos) * rot_dim;
  const int half = rot_dim >> 1;
  const int vec_per_head = head_dim >> 3;
  const int rot_vecs = half >> 3;  // vectors in the first half of the rotated span
  const int64_t page = write_cache ? slot / page_size : 0;
  const int in_page = write_cache ? static_cast<int>(slot % page_size) : 0;

  // ---- q and k heads: rotate ----
  const int n_rot_heads = n_q + n_kv;
  if (!interleaved) {
    // work item = (head, vector index i in [0, rot_vecs)): handles elements [8i, 8i+8) and the partner
    // span at +half.
    for (int w = threadIdx.x; w < n_rot_heads * rot_vecs; w += blockDim.x) {
      const int h = w / rot_vecs, i = w % rot_vecs;
      __nv_bfloat16* base = h < n_q ? q + t * q_stride + static_cast<int64_t>(h) * head_dim
                                    : k + t * k_stride + static_cast<int64_t>(h - n_q) * head_dim;
      uint4* p_lo = reinterpret_cast<uint4*>(base) + i;
      uint4* p_hi = reinterpret_cast<uint4*>(base + half) + i;
      float lo[8], hi[8];
      bf16x8_to_f32(*p_lo, lo);
      bf16x8_to_f32(*p_hi, hi);
      float olo[8], ohi[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float c = cs[i * 8 + j], s = cs[half + i * 8 + j];
        olo[j] = lo[j] * c - hi[j] * s;
        ohi[j] = hi[j] * c + lo[j] * s;
      }
      const uint4 plo = f32_to_bf16x8(olo), phi = f32_to_bf16x8(ohi);
      *p_lo = plo;
      *p_hi = phi;
      if (h >= n_q && write_cache) {
        __nv_bfloat16* dst = k_cache + ((page * n_kv + (h - n_q)) * page_size + in_page) * head_dim;
        reinterpret_cast<uint4*>(dst)[i] = plo;
        reinterpret_cast<uint4*>(dst + half)[i] = phi;
      }
    }
  } else {
    const int rvec = rot_dim >> 3;
    for (int w = threadIdx.x; w < n_rot_heads * rvec; w += blockDim.x) {
      const int h = w / rvec, i = w % rvec;
      __nv_bfloat16* base = h < n_q ? q + t * q_stride + static_cast<int64_t>(h) * head_dim
                                    : k + t * k_stride + static_cast<int64_t>(h - n_q) * head_dim;
      uint4* p = reinterpret_cast<uint4*>(base) + i;
      float e[8], o[8];
      bf16x8_to_f32(*p, e);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int pair = i * 4 + j;
        const float c = cs[pair], s = cs[half + pair];
        o[2 * j] = e[2 * j] * c - e[2 * j + 1] * s;
        o[2 * j + 1] = e[2 * j + 1] * c + e[2 * j] * s;
      }
      const uint4 packed = f32_to_bf16x8(o);
      *p = packed;
      if (h >= n_q && write_cache) {
        __nv_bfloat16* dst = k_cache + ((page * n_kv + (h - n_q)) * page_size + in_page) * head_dim;
        reinterpret_cast<uint4*>(dst)[i] = packed;
      }
    }
  }
  if (!write_cache) return;
  // ---- un-rotated tail of k (rot_dim < head_dim) and all of v: plain copies into the cache ----
  const int tail_vecs = (head_dim - rot_dim) >> 3;
  for (int w = threadIdx.x; w < n_kv * tail_vecs; w += blockDim.x) {
    const int h = w / tail_vecs, i = w % tail_vecs;
    const __nv_bfloat16* src = k + t * k_stride + static_cast<int64_t>(h) * head_dim + rot_dim;
    __nv_bfloat16* dst = k_cache + ((page * n_kv + h) * page_size + in_page) * head_dim + rot_dim;
    reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
  }
  if (v != nullptr && v_cache != nullptr) {
    for (int w = threadIdx.x; w < n_kv * vec_per_head; w += blockDim.x) {
      const int h = w / vec_per_head, i = w % vec_per_head;
      const __nv_bfloat16* src = v + t * v_stride + static_cast<int64_t>(h) * head_dim;
      __nv_bfloat16* dst = v_cache + ((page * n_kv + h) * page_size + in_page) * head_dim;
      reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    }
  }
}

// interleaved = false: row = [gate (ffn) | up (ffn)]. interleaved = true: alternating blocks of 16 gate and 16 up
// columns (the output of a plain GEMM against a weight stacked for the SwiGLU GEMM epilogue).
__global__ void swiglu_kernel(const uint4* __restrict__ gate_up, uint4* __restrict__ out, int rows, int ffn_vecs, bool interleaved) {
  ptx::grid_dep_sync();
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t total = static_cast<int64_t>(rows) * ffn_vecs;
  if (idx >= total) return;
  const int64_t r = idx / ffn_vecs;
  const int c = static_cast<int>(idx % ffn_vecs);
  float g[8], u[8], o[8];
  const int gv = interleaved ? 4 * (c >> 1) + (c & 1) : c;       // 16 columns = 2 vectors per block half
  const int uv = interleaved ? gv + 2 : ffn_vecs + c;
  bf16x8_to_f32(ptx::ld_nc_v4(gate_up + r * 2 * ffn_vecs + gv), g);
  bf16x8_to_f32(ptx::ld_nc_v4(gate_up + r * 2 * ffn_vecs + uv), u);
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = ptx::silu(g[j]) * u[j];
  out[idx] = f32_to_bf16x8(o);
}

// tok[rows[i]] = prev[src[i]] for i < n: the input token of a decode row is the token the previous step sampled for that
// sequence, still on the device when the next step is staged (the host reads it one step later).
__global__ void patch_tokens_kernel(int64_t* __restrict__ tok, const int32_t* __restrict__ rows, const int32_t* __restrict__ src,
                                    const int64_t* __restrict__ prev, int n, int64_t tok_rows, int64_t prev_rows, Status* status) {
  ptx::grid_dep_sync();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t r = rows[i], s2 = src[i];
  if (!B2_ASSERT(status, r >= 0 && r < tok_rows && s2 >= 0 && s2 < prev_rows, kSiteSampling, r, s2)) return;
  tok[r] = prev[s2];
}

__global__ void embedding_kernel(const int64_t* __restrict__ ids, const uint4* __restrict__ table,
                                 uint4* __restrict__ out, int hidden_vecs, int64_t vocab_start, int64_t vocab_rows) {
  ptx::grid_dep_sync();
  const int t = blockIdx.x;
  const int64_t id = ids[t] - vocab_start;
  const bool inside = id >= 0 && id < vocab_rows;
  for (int c = threadIdx.x; c < hidden_vecs; c += blockDim.x) {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (inside) v = ptx::ld_nc_v4(table + id * hidden_vecs + c);
    out[static_cast<size_t>(t) * hidden_vecs + c] = v;
  }
}

__global__ void gather_rows_kernel(const uint4* __restrict__ src, const int64_t* __restrict__ index,
                                   uint4* __restrict__ out, int col_vecs, int64_t rows_src, Status* status) {
  ptx::grid_dep_sync();
  const int r = blockIdx.x;
  const int64_t s = index[r];
  if (!B2_ASSERT(status, s >= 0 && s < rows_src, kSiteKvIndex, s, rows_src)) return;
  for (int c = threadIdx.x; c < col_vecs; c += blockDim.x)
    out[static_cast<size_t>(r) * col_vecs + c] = src[s * col_vecs + c];
}

__global__ void scatter_rows_kernel(const uint4* __restrict__ src, const int64_t* __restrict__ slots, uint4* __restrict__ dst,
                                    int col_vecs, int64_t rows_dst, Status* status) {
  ptx::grid_dep_sync();
  const int r = blockIdx.x;
  const int64_t d = slots[r];
  if (d < 0) return;  // padding row
  if (!B2_ASSERT(status, d < rows_dst, kSiteKvIndex, d, rows_dst)) return;
  for (int c = threadIdx.x; c < col_vecs; c += blockDim.x) dst[d * col_vecs + c] = src[static_cast<size_t>(r) * col_vecs + c];
}

__global__ void copy_pages_kernel(uint4* __restrict__ cache, const int64_t* __restrict__ src_pages,
                                  const int64_t* __restrict__ dst_pages, int64_t page_vecs, int64_t num_pages,
                                  Status* status) {
  ptx::grid_dep_sync();
  const int64_t s = src_pages[blockIdx.y], d = dst_pages[blockIdx.y];
  if (!B2_ASSERT(status, s >= 0 && s < num_pages && d >= 0 && d < num_pages, kSiteKvIndex, s, d)) return;
  for (int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; c < page_vecs;
       c += static_cast<int64_t>(gridDim.x) * blockDim.x)
    cache[d * page_vecs + c] = cache[s * page_vecs + c];
}

template <bool QUANT>
int launch_rmsnorm(const void* x, void* residual, const void* weight, void* out, void* q_out, float* q_scale, int rows,
                   int hidden, float eps, cudaStream_t stream) {
  const int nvec = hidden / 8;
  int vpt = 1;
  while ((nvec + vpt - 1) / vpt > 1024) vpt *= 2;
  if (nvec >= 1024 && vpt == 1) vpt = 2;  // 512 threads x 2 vectors beats 1024 x 1 on occupancy
  int threads = ((nvec + vpt - 1) / vpt + 31) / 32 * 32;
  auto xp = static_cast<const uint4*>(x);
  auto rp = static_cast<uint4*>(residual);
  auto wp = static_cast<const uint4*>(weight);
  auto op = static_cast<uint4*>(out);
  auto qp = static_cast<uint8_t*>(q_out);
  switch (vpt) {
    case 1: launch_pdl(rmsnorm_kernel<1, QUANT>, dim3(rows), dim3(threads), 0, stream, xp, rp, wp, op, qp, q_scale, hidden, eps); break;
    case 2: launch_pdl(rmsnorm_kernel<2, QUANT>, dim3(rows), dim3(threads), 0, stream, xp, rp, wp, op, qp, q_scale, hidden, eps); break;
    case 4: launch_pdl(rmsnorm_kernel<4, QUANT>, dim3(rows), dim3(threads), 0, stream, xp, rp, wp, op, qp, q_scale, hidden, eps); break;
    case 8: launch_pdl(rmsnorm_kernel<8, QUANT>, dim3(rows), dim3(threads), 0, stream, xp, rp, wp, op, qp, q_scale, hidden, eps); break;
    default: return -kBadArgument;
  }
  return 0;
}

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" int b2_rmsnorm_bf16(const void* x, void* residual, const void* weight, void* out, void* q_out,
                               float* q_scale, int rows, int hidden, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hidden <= 0 || hidden % 8 != 0 || hidden > 65536) return -kBadArgument;
  if (q_out != nullptr) {
    if (hidden % 128 != 0 || q_scale == nullptr) return -kBadArgument;
    return launch_rmsnorm<true>(x, residual, weight, out, q_out, q_scale, rows, hidden, eps, stream);
  }
  return launch_rmsnorm<false>(x, residual, weight, out, nullptr, nullptr, rows, hidden, eps, stream);
}

extern "C" int b2_quant_e4m3_1x128(const void* x, void* q_out, float* scale_out, int rows, int cols,
                                   cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (cols % 128 != 0) return -kBadArgument;
  const int64_t groups = static_cast<int64_t>(rows) * (cols / 128);
  const int threads = 256;
  const int64_t blocks = (groups * 16 + threads - 1) / threads;
  launch_pdl(quant_e4m3_1x128_kernel, dim3(static_cast<unsigned>(blocks)), dim3(threads), 0, stream, 
      static_cast<const uint4*>(x), static_cast<uint8_t*>(q_out), scale_out, rows, cols);
  return 0;
}

extern "C" int b2_rope_kvwrite_bf16(void* q, void* k, const void* v, const float* cos_sin, const int32_t* positions,
                                    const int64_t* slots, void* k_cache, void* v_cache, int tokens, int n_q, int n_kv,
                                    int head_dim, int rot_dim, int interleaved, int64_t q_stride, int64_t k_stride,
                                    int64_t v_stride, int page_size, int64_t num_slots, int max_pos, Status* status,
                                    cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (head_dim % 8 != 0 || rot_dim % 16 != 0 || rot_dim > head_dim || q_stride % 8 != 0 || k_stride % 8 != 0 ||
      v_stride % 8 != 0)
    return -kBadArgument;
  launch_pdl(rope_kvwrite_kernel, dim3(tokens), dim3(128), 0, stream, 
      static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), cos_sin,
      positions, slots, static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), n_q, n_kv,
      head_dim, rot_dim, interleaved, q_stride, k_stride, v_stride, page_size, num_slots, max_pos, status);
  return 0;
}

extern "C" int b2_swiglu_bf16(const void* gate_up, void* out, int rows, int ffn, int interleaved, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (ffn % 8 != 0 || (interleaved && ffn % 16 != 0)) return -kBadArgument;
  const int64_t total = static_cast<int64_t>(rows) * (ffn / 8);
  const int threads = 256;
  launch_pdl(swiglu_kernel, dim3(static_cast<unsigned>((total + threads - 1) / threads)), dim3(threads), 0, stream, 
      static_cast<const uint4*>(gate_up), static_cast<uint4*>(out), rows, ffn / 8, interleaved != 0);
  return 0;
}

extern "C" int b2_embedding_bf16(const int64_t* ids, const void* table, void* out, int tokens, int hidden,
                                 int64_t vocab_start, int64_t vocab_rows, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (hidden % 8 != 0) return -kBadArgument;
  const int threads = hidden / 8 >= 256 ? 256 : 128;
  launch_pdl(embedding_kernel, dim3(tokens), dim3(threads), 0, stream, ids, static_cast<const uint4*>(table), static_cast<uint4*>(out),
                                                   hidden / 8, vocab_start, vocab_rows);
  return 0;
}

extern "C" int b2_patch_tokens(int64_t* tok, const int32_t* rows, const int32_t* src, const int64_t* prev, int n, int64_t tok_rows,
                               int64_t prev_rows, Status* status, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (tok == nullptr || rows == nullptr || src == nullptr || prev == nullptr) return -kBadArgument;
  launch_pdl(patch_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, tok, rows, src, prev, n, tok_rows, prev_rows, status);
  return last_launch_rc();
}

extern "C" int b2_gather_rows_bf16(const void* src, const int64_t* index, void* out, int rows_out, int cols,
                                   int64_t rows_src, Status* status, cudaStream_t stream) {
  if (rows_out <= 0) return 0;
  if (cols % 8 != 0) return -kBadArgument;
  launch_pdl(gather_rows_kernel, dim3(rows_out), dim3(128), 0, stream, static_cast<const uint4*>(src), index, static_cast<uint4*>(out),
                                                   cols / 8, rows_src, status);
  return 0;
}

extern "C" int b2_copy_pages(void* cache, const int64_t* src_pages, const int64_t* dst_pages, int n,
                             int64_t page_bytes, int64_t num_pages, Status* status, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (page_bytes % 16 != 0) return -kBadArgument;
  const int64_t vecs = page_bytes / 16;
  const int threads = 256;
  int bx = static_cast<int>((vecs + threads - 1) / threads);
  if (bx > 64) bx = 64;
  launch_pdl(copy_pages_kernel, dim3(dim3(bx, n)), dim3(threads), 0, stream, static_cast<uint4*>(cache), src_pages, dst_pages, vecs,
                                                         num_pages, status);
  return 0;
}

extern "C" int b2_scatter_rows_bf16(const void* src, const int64_t* slots, void* dst, int rows, int cols, int64_t rows_dst,
                                    Status* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (cols % 8 != 0) return -kBadArgument;
  launch_pdl(scatter_rows_kernel, dim3(rows), dim3(128), 0, stream, static_cast<const uint4*>(src), slots, static_cast<uint4*>(dst), cols / 8,
                                                rows_dst, status);
  return 0;
}
