// Host-side n-body integrator: five bodies are far too little work for a GPU. Same constants and update rule as
// examples/nbody.mojo:26-171 (offset momentum, pairwise velocity updates with dt / d^3, then positions).
#include <cmath>
#include "b2/examples.h"

namespace {
constexpr double kPi = 3.141592653589793, kSolarMass = 4 * kPi * kPi, kDays = 365.24;
struct Body { double p[3], v[3], m; };
const Body kInit[5] = {
    {{0, 0, 0}, {0, 0, 0}, kSolarMass},
    {{4.84143144246472090e00, -1.16032004402742839e00, -1.03622044471123109e-01},
     {1.66007664274403694e-03 * kDays, 7.69901118419740425e-03 * kDays, -6.90460016972063023e-05 * kDays}, 9.54791938424326609e-04 * kSolarMass},
    {{8.34336671824457987e00, 4.12479856412430479e00, -4.03523417114321381e-01},
     {-2.76742510726862411e-03 * kDays, 4.99852801234917238e-03 * kDays, 2.30417297573763929e-05 * kDays}, 2.85885980666130812e-04 * kSolarMass},
    {{1.28943695621391310e01, -1.51111514016986312e01, -2.23307578892655734e-01},
     {2.96460137564761618e-03 * kDays, 2.37847173959480950e-03 * kDays, -2.96589568540237556e-05 * kDays}, 4.36624404335156298e-05 * kSolarMass},
    {{1.53796971148509165e01, -2.59193146099879641e01, 1.79258772950371181e-01},
     {2.68067772490389322e-03 * kDays, 1.62824170038242295e-03 * kDays, -9.51592254519715870e-05 * kDays}, 5.15138902046611451e-05 * kSolarMass},
};
double energy(const Body* b) {
  double e = 0;
  for (int i = 0; i < 5; ++i) {
    e += 0.5 * b[i].m * (b[i].v[0] * b[i].v[0] + b[i].v[1] * b[i].v[1] + b[i].v[2] * b[i].v[2]);
    for (int j = i + 1; j < 5; ++j) {
      const double dx = b[i].p[0] - b[j].p[0], dy = b[i].p[1] - b[j].p[1], dz = b[i].p[2] - b[j].p[2];
      e -= b[i].m * b[j].m / std::sqrt(dx * dx + dy * dy + dz * dz);
    }
  }
  return e;
}
}  // namespace

extern "C" double b2_ex_nbody(int64_t steps, double dt, double* energy_before) {
  Body b[5];
  for (int i = 0; i < 5; ++i) b[i] = kInit[i];
  double px = 0, py = 0, pz = 0;
  for (int i = 0; i < 5; ++i) { px += b[i].v[0] * b[i].m; py += b[i].v[1] * b[i].m; pz += b[i].v[2] * b[i].m; }
  b[0].v[0] = -px / kSolarMass; b[0].v[1] = -py / kSolarMass; b[0].v[2] = -pz / kSolarMass;
  if (energy_before) *energy_before = energy(b);
  for (int64_t s = 0; s < steps; ++s) {
    for (int i = 0; i < 5; ++i)
      for (int j = i + 1; j < 5; ++j) {
        const double dx = b[i].p[0] - b[j].p[0], dy = b[i].p[1] - b[j].p[1], dz = b[i].p[2] - b[j].p[2];
        const double d2 = dx * dx + dy * dy + dz * dz;
        const double mag = dt / (d2 * std::sqrt(d2));
        b[i].v[0] -= dx * b[j].m * mag; b[i].v[1] -= dy * b[j].m * mag; b[i].v[2] -= dz * b[j].m * mag;
        b[j].v[0] += dx * b[i].m * mag; b[j].v[1] += dy * b[i].m * mag; b[j].v[2] += dz * b[i].m * mag;
      }
    for (int i = 0; i < 5; ++i) { b[i].p[0] += dt * b[i].v[0]; b[i].p[1] += dt * b[i].v[1]; b[i].p[2] += dt * b[i].v[2]; }
  }
  return energy(b);
}
