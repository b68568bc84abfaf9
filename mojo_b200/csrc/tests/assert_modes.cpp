// One source, compiled once per assertion mode (-DB2_ASSERT_MODE=0..3): prints what a failed check did, so that the
// test can compare the four behaviours. The reference tests its `debug_assert` the same way, one file per mode
// (stdlib/test/builtin/test_debug_assert_mode_none.mojo, ..._warning.mojo, ..._mode_all_error.mojo).
//   none (0): the check is compiled out, the guarded access runs, nothing is recorded
//   warn (1): the failure is recorded, the guarded access still runs
//   safe (2): the failure is recorded, the guarded access is skipped           (the library's build default)
//   all  (3): as safe, and the expensive checks marked B2_ASSERT_ALL are compiled in as well
#include <cstdio>

#include "b2/status.h"

int main() {
  b2::Status cheap{}, costly{}, passing{};
  int ran_cheap = 0, ran_costly = 0, ran_passing = 0;
  const long index = 41, limit = 8;
  if (B2_ASSERT(&cheap, index < limit, b2::kSiteTest, index, limit)) ran_cheap = 1;
  if (B2_ASSERT_ALL(&costly, index < limit, b2::kSiteKvIndex, index, limit)) ran_costly = 1;
  if (B2_ASSERT(&passing, limit < index, b2::kSiteTest, 0, 0)) ran_passing = 1;
  // first failure wins: a second record must not overwrite the first
  b2::status_record(&cheap, b2::kTimeout, b2::kSiteAttn, 1, 2);
  std::printf("mode=%d ran_cheap=%d cheap=%s site=%d a=%lld b=%lld ran_costly=%d costly=%s ran_passing=%d passing=%s\n", B2_ASSERT_MODE,
              ran_cheap, b2::status_code_name(cheap.code), cheap.site, static_cast<long long>(cheap.a), static_cast<long long>(cheap.b),
              ran_costly, b2::status_code_name(costly.code), ran_passing, b2::status_code_name(passing.code));
  return 0;
}
