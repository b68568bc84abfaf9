// Status word + non-trapping assertions.
//
// The reference aborts on a failed check: `abort()` lowers to `llvm.intr.trap`
// (stdlib/src/os/os.mojo:234-275) and `debug_assert` prints block/thread ids and aborts
// (stdlib/src/builtin/debug_assert.mojo:228-350). A trap poisons the CUDA context, so on a device
// shared with other jobs this library never traps: a failed device check writes one record
// {code, site, block, thread, a, b} into a status word in global memory and the kernel finishes
// normally. The host reads the word after the step and turns it into an exception.
#pragma once
#include <cstdint>
#include "b2/config.h"

namespace b2 {

enum StatusCode : int32_t {
  kOk = 0,
  kTimeout = 1,      // a bounded wait ran out (mbarrier, flag, peer signal)
  kAssert = 2,       // B2_ASSERT condition failed
  kOutOfBounds = 3,  // an index computed from runtime metadata was outside its buffer
  kBadArgument = 4,  // host-side validation (never set on device)
  kTooLarge = 5,     // request exceeds a fixed capacity (e.g. static scratch)
};

// Wait/assert sites, so a TIMEOUT says which wait gave up.
enum StatusSite : int32_t {
  kSiteNone = 0,
  kSiteGemmFull = 1,
  kSiteGemmEmpty = 2,
  kSiteGemmTmemFull = 3,
  kSiteGemmTmemEmpty = 4,
  kSiteGemmDrain = 5,
  kSiteSplitK = 6,
  kSitePeerSignal = 7,
  kSiteGridBarrier = 8,
  kSiteAgChunk = 9,
  kSiteRsTile = 10,
  kSiteEpCount = 11,
  kSiteAttn = 12,
  kSiteKvIndex = 13,
  kSiteSampling = 14,
  kSiteTest = 15,
};

struct alignas(16) Status {
  int32_t code;
  int32_t site;
  int32_t block;
  int32_t thread;
  int64_t a;
  int64_t b;
};
static_assert(sizeof(Status) == 32, "Status is 32 bytes");

#if defined(__CUDACC__)
// First failure wins; later ones are dropped so the record stays consistent.
__device__ __forceinline__ void status_record(Status* s, int32_t code, int32_t site, int64_t a = 0,
                                              int64_t b = 0) {
  if (s == nullptr) return;
  if (atomicCAS(&s->code, 0, code) == 0) {
    s->site = site;
    s->block = static_cast<int32_t>(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z));
    s->thread = static_cast<int32_t>(threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z));
    s->a = a;
    s->b = b;
    __threadfence_system();
  }
}

#else
// Host restatement of the device recorder (first failure wins): host-side validation uses the same macro, and the
// assertion modes can be exercised without a device.
inline void status_record(Status* s, int32_t code, int32_t site, int64_t a = 0, int64_t b = 0) {
  if (s == nullptr || s->code != 0) return;
  s->code = code;
  s->site = site;
  s->block = -1;
  s->thread = -1;
  s->a = a;
  s->b = b;
}
#endif  // __CUDACC__

// B2_ASSERT(status, cond, site, a, b): evaluates to `cond`; when false it records and the caller
// is expected to skip the access (`if (!B2_ASSERT(...)) continue;`).
#if B2_ASSERT_MODE == 0
#define B2_ASSERT(status, cond, site, a, b) (true)
#else
#define B2_ASSERT(status, cond, site, a, b) \
  ((cond) ? true : (::b2::status_record((status), ::b2::kAssert, (site), (int64_t)(a), (int64_t)(b)), B2_ASSERT_MODE == 1))
#endif
#if B2_ASSERT_MODE >= 3
#define B2_ASSERT_ALL(status, cond, site, a, b) B2_ASSERT(status, cond, site, a, b)
#else
#define B2_ASSERT_ALL(status, cond, site, a, b) (true)
#endif


inline const char* status_code_name(int32_t c) {
  switch (c) {
    case kOk: return "OK";
    case kTimeout: return "TIMEOUT";
    case kAssert: return "ASSERT";
    case kOutOfBounds: return "OUT_OF_BOUNDS";
    case kBadArgument: return "BAD_ARGUMENT";
    case kTooLarge: return "TOO_LARGE";
    default: return "UNKNOWN";
  }
}

}  // namespace b2
