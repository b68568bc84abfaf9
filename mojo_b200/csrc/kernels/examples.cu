// Compute kernels of the reference's example programs, written as plain CUDA: the three-step matmul
// walk-through (examples/matmul.mojo:103-280: naive -> tiled; the last step is the tcgen05 GEMM of this library),
// Mandelbrot (examples/mandelbrot.mojo:24-69), f32 sum reduction (examples/reduce.mojo:28-51), one Game-of-Life
// generation on a torus (examples/life/gridv2.mojo:97-125) and the sphere ray tracer of
// examples/notebooks/RayTracing.ipynb (cells 16-29). Outputs are plain device buffers; nothing is displayed.
#include <cstdint>
#include <cuda_runtime.h>
#include "b2/api.h"
#include "b2/launch.h"
#include "b2/examples.h"
#include "b2/vec.cuh"

namespace b2 {
namespace {

__global__ void matmul_naive_kernel(const float* a, const float* b, float* c, int M, int N, int K) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x, row = blockIdx.y * blockDim.y + threadIdx.y;
  if (row >= M || col >= N) return;
  float acc = 0.0f;
  for (int k = 0; k < K; ++k) acc = fmaf(a[static_cast<int64_t>(row) * K + k], b[static_cast<int64_t>(k) * N + col], acc);
  c[static_cast<int64_t>(row) * N + col] = acc;
}

constexpr int kTile = 32;
__global__ void matmul_tiled_kernel(const float* a, const float* b, float* c, int M, int N, int K) {
  __shared__ float as[kTile][kTile + 1], bs[kTile][kTile + 1];
  const int col = blockIdx.x * kTile + threadIdx.x, row = blockIdx.y * kTile + threadIdx.y;
  float acc = 0.0f;
  for (int k0 = 0; k0 < K; k0 += kTile) {
    as[threadIdx.y][threadIdx.x] = (row < M && k0 + threadIdx.x < K) ? a[static_cast<int64_t>(row) * K + k0 + threadIdx.x] : 0.0f;
    bs[threadIdx.y][threadIdx.x] = (col < N && k0 + threadIdx.y < K) ? b[static_cast<int64_t>(k0 + threadIdx.y) * N + col] : 0.0f;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kTile; ++k) acc = fmaf(as[threadIdx.y][k], bs[k][threadIdx.x], acc);
    __syncthreads();
  }
  if (row < M && col < N) c[static_cast<int64_t>(row) * N + col] = acc;
}

__global__ void mandelbrot_kernel(int32_t* out, int rows, int cols, int max_iters, float min_x, float max_x, float min_y, float max_y) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x, row = blockIdx.y * blockDim.y + threadIdx.y;
  if (row >= rows || col >= cols) return;
  const float cx = min_x + col * ((max_x - min_x) / cols), cy = min_y + row * ((max_y - min_y) / rows);
  float x = 0.0f, y = 0.0f;
  int iters = 0;
  for (int i = 0; i < max_iters; ++i) {
    // same update order as the reference kernel: y2, y, escape test on the old x, then x
    const float y2 = y * y;
    y = fmaf(x, y + y, cy);
    const bool inside = fmaf(x, x, y2) <= 4.0f;
    x = fmaf(x, x, cx - y2);
    if (!inside) break;
    ++iters;
  }
  out[row * cols + col] = iters;
}

__global__ void reduce_sum_kernel(const float* __restrict__ x, int64_t n, double* __restrict__ out) {
  __shared__ float scratch[33];
  float acc = 0.0f;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x * 4;
  for (int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 3 < n) {
      const float4 v = *reinterpret_cast<const float4*>(x + i);
      acc += (v.x + v.y) + (v.z + v.w);
    } else {
      for (int64_t j = i; j < n; ++j) acc += x[j];
    }
  }
  const float total = block_sum(acc, scratch);
  if (threadIdx.x == 0) atomicAdd(out, static_cast<double>(total));
}

__global__ void life_kernel(const uint8_t* __restrict__ cur, uint8_t* __restrict__ nxt, int rows, int cols) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x, row = blockIdx.y * blockDim.y + threadIdx.y;
  if (row >= rows || col >= cols) return;
  const int up = (row + rows - 1) % rows, dn = (row + 1) % rows, lf = (col + cols - 1) % cols, rt = (col + 1) % cols;
  const int n = cur[up * cols + lf] + cur[up * cols + col] + cur[up * cols + rt] + cur[row * cols + lf] + cur[row * cols + rt] +
                cur[dn * cols + lf] + cur[dn * cols + col] + cur[dn * cols + rt];
  nxt[row * cols + col] = ((n | cur[row * cols + col]) == 3) ? 1 : 0;  // the reference's `num_neighbors | cell == 3` rule
}

struct V3 { float x, y, z; };
__device__ __forceinline__ V3 operator+(V3 a, V3 b) { return {a.x + b.x, a.y + b.y, a.z + b.z}; }
__device__ __forceinline__ V3 operator-(V3 a, V3 b) { return {a.x - b.x, a.y - b.y, a.z - b.z}; }
__device__ __forceinline__ V3 operator*(V3 a, float s) { return {a.x * s, a.y * s, a.z * s}; }
__device__ __forceinline__ float dot(V3 a, V3 b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
__device__ __forceinline__ V3 normalize(V3 a) { return a * (1.0f / sqrtf(dot(a, a))); }

__constant__ B2Scene c_scene;

__device__ bool sphere_hit(const B2Sphere& s, V3 orig, V3 dir, float& dist) {
  const V3 L = orig - V3{s.cx, s.cy, s.cz};
  const float a = dot(dir, dir), b = 2.0f * dot(dir, L), c = dot(L, L) - s.radius * s.radius;
  const float disc = b * b - 4.0f * a * c;
  if (disc < 0.0f) return false;
  if (disc == 0.0f) { dist = -b / 2.0f * a; return true; }
  const float q = b > 0.0f ? -0.5f * (b + sqrtf(disc)) : -0.5f * (b - sqrtf(disc));
  float t0 = q / a;
  const float t1 = c / q;
  if (t0 > t1) t0 = t1;
  if (t0 < 0.0f) { t0 = t1; if (t0 < 0.0f) return false; }
  dist = t0;
  return true;
}

__global__ void raytrace_kernel(float* __restrict__ img, const float* __restrict__ bg, int H, int W, int bg_h, int bg_w) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x, row = blockIdx.y * blockDim.y + threadIdx.y;
  if (row >= H || col >= W) return;
  const float y = -((2.0f * row + 1.0f) / H - 1.0f);
  const float x = ((2.0f * col + 1.0f) / W - 1.0f) * W / H;
  const V3 dir = normalize(V3{x, y, -1.0f}), orig{0.0f, 0.0f, 0.0f};
  float best = INFINITY;
  int hit = -1;
  for (int i = 0; i < c_scene.n_spheres; ++i) {
    float d = 0.0f;
    if (sphere_hit(c_scene.spheres[i], orig, dir, d) && d < best) { best = d; hit = i; }
  }
  V3 out;
  if (hit < 0) {
    if (bg != nullptr) {
      const int bc = static_cast<int>((1.0f + dir.x) * 0.5f * (bg_w - 1)), br = static_cast<int>((1.0f + dir.y) * 0.5f * (bg_h - 1));
      const float* p = bg + (static_cast<int64_t>(br) * bg_w + bc) * 3;
      out = {p[0], p[1], p[2]};
    } else {
      out = {0.02f, 0.02f, 0.02f};
    }
  } else {
    const B2Sphere& s = c_scene.spheres[hit];
    const V3 point = orig + dir * best;
    const V3 N = normalize(point - V3{s.cx, s.cy, s.cz});
    float diffuse = 0.0f, spec = 0.0f;
    for (int i = 0; i < c_scene.n_lights; ++i) {
      const B2Light& l = c_scene.lights[i];
      const V3 ld = normalize(V3{l.x, l.y, l.z} - point);
      diffuse += l.intensity * fmaxf(dot(ld, N), 0.0f);
      const V3 I = ld * -1.0f;
      const V3 refl = I - N * (dot(I, N) * 2.0f);
      spec += powf(fmaxf(-dot(refl, dir), 0.0f), s.specular) * l.intensity;
    }
    out = V3{s.r, s.g, s.b} * (diffuse * s.albedo0) + V3{1.0f, 1.0f, 1.0f} * (spec * s.albedo1);
    const float mx = fmaxf(out.x, fmaxf(out.y, out.z));
    if (mx > 1.0f) out = out * (1.0f / mx);
  }
  float* o = img + (static_cast<int64_t>(row) * W + col) * 3;
  o[0] = out.x; o[1] = out.y; o[2] = out.z;
}

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" int b2_ex_matmul(const float* a, const float* b, float* c, int M, int N, int K, int variant, cudaStream_t stream) {
  if (variant == 0) {
    matmul_naive_kernel<<<dim3((N + 15) / 16, (M + 15) / 16), dim3(16, 16), 0, stream>>>(a, b, c, M, N, K);
  } else {
    matmul_tiled_kernel<<<dim3((N + kTile - 1) / kTile, (M + kTile - 1) / kTile), dim3(kTile, kTile), 0, stream>>>(a, b, c, M, N, K);
  }
  return last_launch_rc();
}
extern "C" int b2_ex_mandelbrot(int32_t* out, int rows, int cols, int max_iters, float min_x, float max_x, float min_y, float max_y,
                                cudaStream_t stream) {
  mandelbrot_kernel<<<dim3((cols + 31) / 32, (rows + 7) / 8), dim3(32, 8), 0, stream>>>(out, rows, cols, max_iters, min_x, max_x, min_y, max_y);
  return last_launch_rc();
}
extern "C" int b2_ex_reduce_sum(const float* x, int64_t n, double* out, cudaStream_t stream) {
  if (cudaMemsetAsync(out, 0, sizeof(double), stream) != cudaSuccess) return -kBadArgument;
  int blocks = static_cast<int>((n / 4 + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  reduce_sum_kernel<<<blocks, 256, 0, stream>>>(x, n, out);
  return last_launch_rc();
}
extern "C" int b2_ex_life(const uint8_t* cur, uint8_t* nxt, int rows, int cols, cudaStream_t stream) {
  life_kernel<<<dim3((cols + 31) / 32, (rows + 7) / 8), dim3(32, 8), 0, stream>>>(cur, nxt, rows, cols);
  return last_launch_rc();
}
extern "C" int b2_ex_raytrace(float* img, const float* bg, int H, int W, int bg_h, int bg_w, const B2Scene* scene, cudaStream_t stream) {
  if (scene == nullptr || scene->n_spheres > 8 || scene->n_lights > 4) return -kBadArgument;
  if (cudaMemcpyToSymbolAsync(c_scene, scene, sizeof(B2Scene), 0, cudaMemcpyHostToDevice, stream) != cudaSuccess) return -kBadArgument;
  raytrace_kernel<<<dim3((W + 15) / 16, (H + 15) / 16), dim3(16, 16), 0, stream>>>(img, bg, H, W, bg_h, bg_w);
  return last_launch_rc();
}
