// C API of the example kernels (csrc/kernels/examples.cu) and the host n-body integrator (csrc/runtime/nbody.cpp).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

struct B2Sphere { float cx, cy, cz, radius, r, g, b, albedo0, albedo1, specular; };
struct B2Light { float x, y, z, intensity; };
struct B2Scene { int n_spheres, n_lights; struct B2Sphere spheres[8]; struct B2Light lights[4]; };

// variant 0: one thread per output, global loads only; variant 1: 32x32 shared-memory tiles. a [M,K], b [K,N], c [M,N] f32.
int b2_ex_matmul(const float* a, const float* b, float* c, int M, int N, int K, int variant, cudaStream_t stream);
int b2_ex_mandelbrot(int32_t* out, int rows, int cols, int max_iters, float min_x, float max_x, float min_y, float max_y, cudaStream_t stream);
int b2_ex_reduce_sum(const float* x, int64_t n, double* out, cudaStream_t stream);
int b2_ex_life(const uint8_t* cur, uint8_t* nxt, int rows, int cols, cudaStream_t stream);
// img f32 [H, W, 3]; bg optional f32 [bg_h, bg_w, 3] looked up by ray direction for rays that hit nothing.
int b2_ex_raytrace(float* img, const float* bg, int H, int W, int bg_h, int bg_w, const struct B2Scene* scene, cudaStream_t stream);
// Five-body solar system (Sun, Jupiter, Saturn, Uranus, Neptune), symplectic Euler steps of `dt`; returns the energy.
double b2_ex_nbody(int64_t steps, double dt, double* energy_before);

#ifdef __cplusplus
}
#endif
