// Build-time configuration for the sm_100a kernel library.
//
// Plays the role of the reference's compile-time defines (`mojo -D KEY=VAL`, read by
// stdlib/src/sys/param_env.mojo:44-187 and stdlib/src/sys/_build.mojo:18-62): every knob is an
// nvcc `-D` macro with a default, and nothing else in the tree reads the environment at compile time.
#pragma once

// Assertion modes mirror stdlib/src/builtin/debug_assert.mojo:35-57 (ASSERT=none|warn|safe|all).
//   0 none : checks compiled out
//   1 warn : failed check is recorded in the status word, execution continues
//   2 safe : cheap checks (bounds computed from runtime metadata) recorded, the offending access is skipped
//   3 all  : safe + expensive checks
#ifndef B2_ASSERT_MODE
#define B2_ASSERT_MODE 2
#endif

// Single compile target. There is no fallback ladder (the reference gates on sm_80/sm_90a strings,
// stdlib/src/sys/info.mojo:423-480; here only Blackwell sm_100a exists).
#if defined(__CUDA_ARCH__)
#if __CUDA_ARCH__ != 1000
#error "mojo_b200 kernels are written for sm_100a only"
#endif
#endif

#ifndef B2_DEBUG
#define B2_DEBUG 0
#endif

// Device-side wait limits. Every spin in this library is bounded twice: by an iteration count and by
// a %globaltimer deadline, whichever is hit first.
#ifndef B2_WAIT_MAX_ITERS
#define B2_WAIT_MAX_ITERS (1u << 26)
#endif
#ifndef B2_WAIT_TIMEOUT_NS
#define B2_WAIT_TIMEOUT_NS 2000000000ull  // 2 s for waits inside one kernel
#endif
#ifndef B2_PEER_WAIT_TIMEOUT_NS
#define B2_PEER_WAIT_TIMEOUT_NS 1000000000ull  // 1 s default for waits on another GPU
#endif

namespace b2 {
constexpr int kNumSMs = 148;          // B200: 2 dies x 74 SMs
constexpr int kMaxSmemPerCta = 232448;  // 227 KiB opt-in
constexpr int kTmemColumns = 512;     // 128 lanes x 512 32-bit columns per SM
constexpr int kWarpSize = 32;
}  // namespace b2
